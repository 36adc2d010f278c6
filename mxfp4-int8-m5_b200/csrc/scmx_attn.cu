// Batch-1 decode attention over a preallocated KV cache with the sequence length read on the device, so that a whole
// decode step (GEMVs, row kernels, this kernel) can be replayed from one CUDA graph while the position advances.
// The reference leaves this step to MLX's scaled_dot_product_attention (e2e/decode.py:103, e2e/fused_qwen3.py:197-203);
// it is outside the W4A8 arithmetic and carries no bit-parity claim: float32 online softmax, one bf16 rounding at the end.
#include "scmx_attn_core.cuh"

namespace scmx {

struct AttnArgs {
    const uint16_t* q;       // bf16 [hq, d]
    const uint16_t* k;       // bf16 [hk, cap, d]
    const uint16_t* v;
    const int32_t* pos_dev;  // null, or the index of the newest position: T = pos_dev[0] + 1
    float* part;             // f32 [hq, nsplit, d + 2]: unnormalized output, running max (log2 domain), running sum
    int32_t* counters;       // int32 [hk], zero before the first call; the kernel leaves them zero
    uint16_t* out;           // bf16 [hq * d]
    int64_t cap;
    int t_static, hq, hk, nsplit;
    float scale;
};

template <int G, int D>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(const AttnArgs a) {
    __shared__ AttnSmem<G, D> sm;
    __shared__ int s_ticket;
    pdl_launch_dependents();
    pdl_wait();
    const int kvh = blockIdx.x, split = blockIdx.y, tid = threadIdx.x;
    int64_t T = a.pos_dev ? (int64_t)a.pos_dev[0] + 1 : (int64_t)a.t_static;
    T = T < 1 ? 1 : (T > a.cap ? a.cap : T);
    int64_t chunk;
    int active;
    attn_chunking(T, a.nsplit, chunk, active);
    if (split >= active) return;
    const int64_t t0 = (int64_t)split * chunk, t1 = t0 + chunk < T ? t0 + chunk : T;
    constexpr int stride = D + 2;
    attn_split<G, D>(a.q + (size_t)kvh * G * D, a.k + (size_t)kvh * a.cap * D, a.v + (size_t)kvh * a.cap * D, t0, t1, -1, nullptr,
                     nullptr, a.scale, a.part + ((size_t)kvh * G * a.nsplit + split) * stride, (size_t)a.nsplit * stride, sm);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(a.counters + kvh, 1);
    __syncthreads();
    if (s_ticket != active - 1) return;
    __threadfence();
    // the last CTA of this kv head combines the splits
    attn_combine_cta<G, D>(a.part + (size_t)kvh * G * a.nsplit * stride, a.nsplit, active, a.out + (size_t)kvh * G * D, sm);
    if (tid == 0) a.counters[kvh] = 0;
}

template <int G>
static cudaError_t launch_attn(const AttnArgs& a, int d, cudaStream_t st) {
    const dim3 grid((unsigned)a.hk, (unsigned)a.nsplit), block(AD_THREADS);
    if (d == 128) return launch_pdl(attn_decode_kernel<G, 128>, grid, block, 0, st, a);
    return launch_pdl(attn_decode_kernel<G, 64>, grid, block, 0, st, a);
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_attn_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, int64_t capacity,
                                const int32_t* pos_dev, int64_t n_pos, float scale, int hq, int hk, int d, int nsplit,
                                float* partials, int32_t* counters, uint16_t* out, void* stream) {
    SCMX_REQUIRE(q && k_cache && v_cache && partials && counters && out, SCMX_EINVAL, "attn_decode: null buffer");
    SCMX_REQUIRE(d == 64 || d == 128, SCMX_EINVAL, "attn_decode: head size %d (64 or 128)", d);
    SCMX_REQUIRE(hq > 0 && hk > 0 && hq % hk == 0, SCMX_EINVAL, "attn_decode: hq=%d hk=%d", hq, hk);
    const int G = hq / hk;
    SCMX_REQUIRE(G == 1 || G == 2 || G == 4, SCMX_ELIMIT, "attn_decode: %d query heads per key/value head (1, 2 or 4)", G);
    SCMX_REQUIRE(nsplit >= 1 && nsplit <= 32, SCMX_EINVAL, "attn_decode: nsplit=%d (1..32)", nsplit);
    SCMX_REQUIRE(capacity >= 1 && (pos_dev != nullptr || (n_pos >= 1 && n_pos <= capacity)), SCMX_EINVAL,
                 "attn_decode: %lld positions in a cache of %lld", (long long)n_pos, (long long)capacity);
    SCMX_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, SCMX_EINVAL, "attn_decode: cache not 16-byte aligned");
    AttnArgs a;
    a.q = q; a.k = k_cache; a.v = v_cache; a.pos_dev = pos_dev; a.part = partials; a.counters = counters; a.out = out;
    a.cap = capacity; a.t_static = (int)n_pos; a.hq = hq; a.hk = hk; a.nsplit = nsplit; a.scale = scale;
    cudaError_t e = G == 1 ? launch_attn<1>(a, d, (cudaStream_t)stream)
                  : G == 2 ? launch_attn<2>(a, d, (cudaStream_t)stream) : launch_attn<4>(a, d, (cudaStream_t)stream);
    SCMX_PDL_OK("attn_decode_kernel", e);
    return SCMX_OK;
}
