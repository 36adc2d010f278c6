// q/k/v epilogue between the fused q|k|v projection and attention: RMSNorm of q and k (per head, or over the whole
// q / k vector), optional rotary embedding, head-major outputs that may be rows of a KV cache.
// Replaces qkv_epilogue_headnorm, qkv_headnorm_y and qkv_fullnorm_y (e2e/sc_kernels.py:333-423,597-637); the rotary
// step and the cache append are what the reference leaves to MLX (e2e/fused_qwen3.py:197-203).
#include "scmx_common.cuh"

namespace scmx {

struct QkvArgs {
    const void* src;          // bf16 y [L, ntot] or int32 acc [L, ntot]
    const float* xscale;      // [L]     (acc input only)
    const float* wscale;      // [ntot]  (acc input only)
    const uint16_t* qn;       // bf16 [d] (per head) or [hq*d] (full)
    const uint16_t* kn;       // bf16 [d] or [hk*d]
    const float* inv_freq;    // f32 [d/2] or null: no rotary embedding
    const int32_t* pos_dev;   // null, or one int32 added to pos0 and kv_row0 (a step counter kept on the device)
    const float* rope_cs;     // null, or a table f32 [rope_rows, d]: cos (d/2) then sin (d/2) of position * inv_freq
    int64_t rope_rows;
    uint16_t *q, *k, *v;
    int64_t q_hs, kv_hs, kv_row0, pos0;
    float eps;
    int hq, hk, d, d_shift, full;
};

// One CTA per token row.  Shared memory: the bf16-rounded row as float [ntot], 1/rms per q and k head, cos/sin [d/2] each.
template <bool FROM_ACC>
__global__ void __launch_bounds__(256) qkv_norm_kernel(const QkvArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ double red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t step = a.pos_dev ? (int64_t)a.pos_dev[0] : 0;
    const int64_t kv_row = a.kv_row0 + step + row;
    const int d = a.d, nh = a.hq + a.hk, ntot = (a.hq + 2 * a.hk) * d, half = d >> 1;
    float* vals = reinterpret_cast<float*>(smem_raw);
    float* inv = vals + ntot;
    float* cs = inv + nh;
    float* sn = cs + half;

    if (FROM_ACC) {
        const int32_t* acc = static_cast<const int32_t*>(a.src) + (int64_t)row * ntot;
        const float xs = a.xscale[row];
        for (int e = tid; e < ntot; e += 256) vals[e] = scale_acc(acc[e], xs, a.wscale[e]);
    } else {
        const uint32_t* y = reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(a.src) + (int64_t)row * ntot);
        for (int e = tid; e < (ntot >> 1); e += 256) {
            const uint32_t w = y[e];
            vals[2 * e] = __uint_as_float(w << 16);
            vals[2 * e + 1] = __uint_as_float(w & 0xFFFF0000u);
        }
    }
    if (a.inv_freq != nullptr) {
        const int64_t pos = a.pos0 + step + row;
        for (int i = tid; i < half; i += 256) {
            if (a.rope_cs != nullptr && pos < a.rope_rows) {    // the same values, computed once on the host side
                cs[i] = a.rope_cs[pos * d + i];
                sn[i] = a.rope_cs[pos * d + half + i];
            } else {
                const float ang = __fmul_rn((float)pos, a.inv_freq[i]);
                double s, c;
                sincos((double)ang, &s, &c);
                cs[i] = (float)c;
                sn[i] = (float)s;
            }
        }
    }
    __syncthreads();

    if (!a.full) {
        // 8 lanes per head, 4 heads per warp at a time (the trip count is uniform over the warp)
        const int sub = lane >> 3, l8 = lane & 7;
        for (int g0 = warp * 4; g0 < nh; g0 += 32) {
            const int g = g0 + sub;
            double ss = 0.0;
            if (g < nh)
                for (int i = l8; i < d; i += 8) {
                    const double x = (double)vals[g * d + i];
                    ss += x * x;
                }
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            ss += __shfl_xor_sync(0xffffffffu, ss, 4);
            if (g < nh && l8 == 0) inv[g] = rms_inverse(ss, d, a.eps);
        }
    } else {
        for (int part = 0; part < 2; ++part) {
            const int h0 = part ? a.hq : 0, hn = part ? a.hk : a.hq;
            double ss = 0.0;
            for (int i = tid; i < hn * d; i += 256) {
                const double x = (double)vals[h0 * d + i];
                ss += x * x;
            }
            ss = block_sum(ss, red);
            const float r = rms_inverse(ss, hn * d, a.eps);
            for (int g = tid; g < hn; g += 256) inv[h0 + g] = r;
        }
    }
    __syncthreads();

    // normalized value of element e of the row: T(w * T(x * inv)) for q and k, x itself for v
    auto normed = [&](int e) -> float {
        const int g = e >> a.d_shift, dd = e & (d - 1);
        const float x = vals[e];
        if (g >= nh) return x;
        const bool isq = g < a.hq;
        const uint16_t* w = isq ? a.qn : a.kn;
        const int wi = a.full ? (isq ? e : e - a.hq * d) : dd;
        return rbf(__fmul_rn(bf16_to_f32(w[wi]), rbf(__fmul_rn(x, inv[g]))));
    };
    auto rotated = [&](int e, float self) -> float {
        const int g = e >> a.d_shift, dd = e & (d - 1);
        if (a.inv_freq == nullptr || g >= nh) return self;
        const bool lo = dd < half;
        const float other = normed(lo ? e + half : e - half);
        const int i = lo ? dd : dd - half;
        // lo: x1 cos - x2 sin with (x1, x2) = (self, other); hi: x1 sin + x2 cos with (x1, x2) = (other, self)
        return lo ? rbf(__fsub_rn(__fmul_rn(self, cs[i]), __fmul_rn(other, sn[i])))
                  : rbf(__fadd_rn(__fmul_rn(other, sn[i]), __fmul_rn(self, cs[i])));
    };
    for (int e = 2 * tid; e < ntot; e += 512) {
        const int g = e >> a.d_shift, dd = e & (d - 1);
        const float y0 = rotated(e, normed(e)), y1 = rotated(e + 1, normed(e + 1));
        uint16_t* out;
        if (g >= a.hq && kv_row >= a.kv_hs) continue;   // a device-side step beyond the cache: drop the row
        if (g < a.hq) out = a.q + ((int64_t)g * a.q_hs + row) * d;
        else if (g < nh) out = a.k + ((int64_t)(g - a.hq) * a.kv_hs + kv_row) * d;
        else out = a.v + ((int64_t)(g - nh) * a.kv_hs + kv_row) * d;
        *reinterpret_cast<uint32_t*>(out + dd) = (uint32_t)f32_to_bf16(y0) | ((uint32_t)f32_to_bf16(y1) << 16);
    }
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_qkv_norm(const void* src, int src_is_acc, const float* xscale, const float* wscale, const uint16_t* qn,
                             const uint16_t* kn, float eps, int64_t L, int hq, int hk, int d, int full, const float* inv_freq,
                             const float* rope_table, int64_t rope_rows, int64_t pos0, const int32_t* pos_dev, uint16_t* q, int64_t q_head_stride, uint16_t* k, uint16_t* v,
                             int64_t kv_head_stride, int64_t kv_row0, void* stream) {
    SCMX_REQUIRE(L >= 0 && hq > 0 && hk > 0, SCMX_EINVAL, "qkv_norm: L=%lld hq=%d hk=%d", (long long)L, hq, hk);
    SCMX_REQUIRE(d >= 8 && (d & (d - 1)) == 0, SCMX_EINVAL, "qkv_norm: head size %d must be a power of two >= 8", d);
    SCMX_REQUIRE(q_head_stride >= L && kv_head_stride >= kv_row0 + L && kv_row0 >= 0 && pos0 >= 0, SCMX_EINVAL,
                 "qkv_norm: head strides (%lld, %lld) do not hold %lld rows from row %lld", (long long)q_head_stride,
                 (long long)kv_head_stride, (long long)L, (long long)kv_row0);
    SCMX_REQUIRE(!src_is_acc || (xscale != nullptr && wscale != nullptr), SCMX_EINVAL, "qkv_norm: int32 input needs xscale and wscale");
    SCMX_REQUIRE(src && qn && kn && q && k && v, SCMX_EINVAL, "qkv_norm: null buffer");
    const int64_t ntot = (int64_t)(hq + 2 * hk) * d;
    const size_t smem = (size_t)ntot * 4 + (size_t)(hq + hk) * 4 + (size_t)d * 4;
    SCMX_REQUIRE(smem <= 48 * 1024, SCMX_ELIMIT, "qkv_norm: a row of %lld values does not fit the 48 KB of shared memory", (long long)ntot);
    if (L == 0) return SCMX_OK;
    QkvArgs a;
    a.src = src; a.xscale = xscale; a.wscale = wscale; a.qn = qn; a.kn = kn; a.inv_freq = inv_freq; a.pos_dev = pos_dev;
    a.rope_cs = rope_table; a.rope_rows = rope_table ? rope_rows : 0;
    a.q = q; a.k = k; a.v = v;
    a.q_hs = q_head_stride; a.kv_hs = kv_head_stride; a.kv_row0 = kv_row0; a.pos0 = pos0;
    a.eps = eps; a.hq = hq; a.hk = hk; a.d = d; a.full = full ? 1 : 0;
    a.d_shift = 0;
    while ((1 << a.d_shift) < d) ++a.d_shift;
    if (src_is_acc)
        SCMX_PDL_OK("qkv_norm_kernel", launch_pdl(qkv_norm_kernel<true>, dim3((unsigned)L), dim3(256), smem, (cudaStream_t)stream, a));
    else
        SCMX_PDL_OK("qkv_norm_kernel", launch_pdl(qkv_norm_kernel<false>, dim3((unsigned)L), dim3(256), smem, (cudaStream_t)stream, a));
    return SCMX_OK;
}
