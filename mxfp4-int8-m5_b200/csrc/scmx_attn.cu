// Batch-1 decode attention over a preallocated KV cache with the sequence length read on the device, so that a whole
// decode step (GEMVs, row kernels, this kernel) can be replayed from one CUDA graph while the position advances.
// The reference leaves this step to MLX's scaled_dot_product_attention (e2e/decode.py:103, e2e/fused_qwen3.py:197-203);
// it is outside the W4A8 arithmetic and carries no bit-parity claim: float32 online softmax, one bf16 rounding at the end.
#include "scmx_common.cuh"

namespace scmx {

constexpr int AD_THREADS = 128;        // 4 warps x 4 position slots x 8 lanes per position
constexpr int AD_MIN_CHUNK = 64;
constexpr float LOG2E = 1.4426950408889634f;

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

// merge (m2, l2, a2) into (m, l, a): two partial softmax states over disjoint positions
template <int E>
__device__ __forceinline__ void merge_state(float& m, float& l, float (&a)[E], float m2, float l2, const float (&a2)[E]) {
    const float mn = fmaxf(m, m2);
    if (mn == -INFINITY) return;
    const float c1 = exp2f(m - mn), c2 = exp2f(m2 - mn);
    l = l * c1 + l2 * c2;
#pragma unroll
    for (int i = 0; i < E; ++i) a[i] = a[i] * c1 + a2[i] * c2;
    m = mn;
}

template <int G, int D>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(const AttnArgs a) {
    constexpr int E = D / 8;                  // elements per lane
    __shared__ float s_acc[4][G][D];
    __shared__ float s_ml[4][G][2];
    __shared__ int s_ticket;
    pdl_launch_dependents();
    pdl_wait();
    const int kvh = blockIdx.x, split = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, slot = lane >> 3, l8 = lane & 7;
    int64_t T = a.pos_dev ? (int64_t)a.pos_dev[0] + 1 : (int64_t)a.t_static;
    T = T < 1 ? 1 : (T > a.cap ? a.cap : T);
    // at least AD_MIN_CHUNK positions per CTA: a short sequence uses the first few splits only, the rest leave at once
    int64_t chunk = (T + a.nsplit - 1) / a.nsplit;
    chunk = chunk < AD_MIN_CHUNK ? AD_MIN_CHUNK : ((chunk + 15) & ~(int64_t)15);
    const int active = (int)((T + chunk - 1) / chunk);
    if (split >= active) return;
    const int64_t t0 = (int64_t)split * chunk, t1 = t0 + chunk < T ? t0 + chunk : T;

    float qf[G][E], acc[G][E], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint16_t* qp = a.q + (size_t)(kvh * G + g) * D + l8 * E;
#pragma unroll
        for (int i = 0; i < E; ++i) {
            qf[g][i] = bf16_to_f32(qp[i]) * (a.scale * LOG2E);
            acc[g][i] = 0.0f;
        }
        m[g] = -INFINITY;
        l[g] = 0.0f;
    }
    const uint16_t* kb = a.k + (size_t)kvh * a.cap * D + l8 * E;
    const uint16_t* vb = a.v + (size_t)kvh * a.cap * D + l8 * E;
    // the trip count is uniform over the warp (the shuffles below need every lane); slots past the end are masked
    for (int64_t tb = t0 + warp * 4; tb < t1; tb += 16) {
        const int64_t t = tb + slot;
        const bool valid = t < t1;
        float kf[E], vf[E];
#pragma unroll
        for (int c = 0; c < E / 8; ++c) {
            uint4 kw = make_uint4(0, 0, 0, 0), vw = make_uint4(0, 0, 0, 0);
            if (valid) {
                kw = *reinterpret_cast<const uint4*>(kb + t * D + 8 * c);
                vw = *reinterpret_cast<const uint4*>(vb + t * D + 8 * c);
            }
            const uint32_t ku[4] = {kw.x, kw.y, kw.z, kw.w}, vu[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                kf[8 * c + 2 * i] = __uint_as_float(ku[i] << 16);
                kf[8 * c + 2 * i + 1] = __uint_as_float(ku[i] & 0xFFFF0000u);
                vf[8 * c + 2 * i] = __uint_as_float(vu[i] << 16);
                vf[8 * c + 2 * i + 1] = __uint_as_float(vu[i] & 0xFFFF0000u);
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < E; ++i) s = fmaf(qf[g][i], kf[i], s);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (valid) {
                const float mn = fmaxf(m[g], s);
                const float corr = exp2f(m[g] - mn), p = exp2f(s - mn);
                l[g] = l[g] * corr + p;
#pragma unroll
                for (int i = 0; i < E; ++i) acc[g][i] = acc[g][i] * corr + p * vf[i];
                m[g] = mn;
            }
        }
    }
    // merge the 4 position slots of a warp
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m[g], off), l2 = __shfl_xor_sync(0xffffffffu, l[g], off);
            float a2[E];
#pragma unroll
            for (int i = 0; i < E; ++i) a2[i] = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
            merge_state<E>(m[g], l[g], acc[g], m2, l2, a2);
        }
    }
    if (slot == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int i = 0; i < E; ++i) s_acc[warp][g][l8 * E + i] = acc[g][i];
            if (l8 == 0) {
                s_ml[warp][g][0] = m[g];
                s_ml[warp][g][1] = l[g];
            }
        }
    }
    __syncthreads();
    // merge the 4 warps; thread e < D owns output element e of every q head of this kv head
    const int stride = D + 2;
    for (int g = 0; g < G; ++g) {
        float mm = -INFINITY;
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_ml[w][g][0]);
        float ll = 0.0f, av = 0.0f;
        for (int w = 0; w < 4; ++w) {
            const float c = mm == -INFINITY ? 0.0f : exp2f(s_ml[w][g][0] - mm);
            ll += s_ml[w][g][1] * c;
            if (tid < D) av += s_acc[w][g][tid] * c;
        }
        float* p = a.part + ((size_t)(kvh * G + g) * a.nsplit + split) * stride;
        if (tid < D) p[tid] = av;
        if (tid == 0) {
            p[D] = mm;
            p[D + 1] = ll;
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(a.counters + kvh, 1);
    __syncthreads();
    if (s_ticket != active - 1) return;
    __threadfence();
    // the last CTA of this kv head combines the splits
    for (int g = 0; g < G; ++g) {
        const float* p = a.part + (size_t)(kvh * G + g) * a.nsplit * stride;
        float mm = -INFINITY;
        for (int s = 0; s < active; ++s) mm = fmaxf(mm, __ldcg(p + s * stride + D));
        float ll = 0.0f, av = 0.0f;
        for (int s = 0; s < active; ++s) {
            const float ms = __ldcg(p + s * stride + D);
            const float c = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
            ll += __ldcg(p + s * stride + D + 1) * c;
            if (tid < D) av += __ldcg(p + s * stride + tid) * c;
        }
        if (tid < D) a.out[(size_t)(kvh * G + g) * D + tid] = f32_to_bf16(av / ll);
    }
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
    SCMX_REQUIRE(nsplit >= 1 && nsplit <= 64, SCMX_EINVAL, "attn_decode: nsplit=%d", nsplit);
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
