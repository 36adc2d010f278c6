// SC-MXFP4 quantizer + packer on the GPU, in float64, bit-compatible with the reference's NumPy pipeline
// (sim/mx_int8.py:39-109 via sim/make_testcase.py:26-44 and e2e/sc_format.py:93-111).
//
// One CTA per weight row, one thread per 32-wide block (looping when a row has more blocks than threads):
//   1. e0 = floor(log2 amax) - 2; candidates e0-1 then e0+1 replace the running best only when their squared error
//      is strictly smaller.  The 32 squared errors are summed in the order NumPy's pairwise reduction uses for a
//      contiguous axis of 32 doubles (eight strided partial sums, then a fixed tree) with no fused multiply-adds,
//      so near-ties resolve exactly as in the reference.
//   2. spread constraint: e = max(e, rowmax(e) - 3) (all-zero row: rowmax = 0); E_lo = rowmin(e); shift = e - E_lo.
//   3. E2M1 rounding with exact ties toward the smaller magnitude; nibble = sign << 3 | idx, eight per word;
//      2-bit shifts four per byte; wscale = 2^(E_lo - 1).
#include <limits.h>
#include "scmx_common.cuh"

namespace scmx {

__device__ __forceinline__ int e2m1_idx(double a) {
    // number of midpoints {.25,.75,1.25,1.75,2.5,3.5,5} strictly below a (np.searchsorted side='left')
    return (a > 0.25) + (a > 0.75) + (a > 1.25) + (a > 1.75) + (a > 2.5) + (a > 3.5) + (a > 5.0);
}
__device__ __forceinline__ int e2m1_x2(int idx) { return (int)((0xC8643210u >> (4 * idx)) & 0xFu); }

__device__ __forceinline__ double block_sq_err(const double (&b)[32], int e) {
    const double s = scalbn(1.0, e), si = scalbn(1.0, -e);
    double r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const double x = b[j + 8 * i];
            const double t = __dmul_rn(x, si);
            const double mag = 0.5 * (double)e2m1_x2(e2m1_idx(fabs(t)));
            const double v = t < 0.0 ? -mag : mag;
            const double d = __dsub_rn(__dmul_rn(v, s), x);
            const double sq = __dmul_rn(d, d);
            r[j] = (i == 0) ? sq : __dadd_rn(r[j], sq);
        }
    }
    return __dadd_rn(__dadd_rn(__dadd_rn(r[0], r[1]), __dadd_rn(r[2], r[3])),
                     __dadd_rn(__dadd_rn(r[4], r[5]), __dadd_rn(r[6], r[7])));
}

template <typename T> __device__ __forceinline__ double to_f64(T v);
template <> __device__ __forceinline__ double to_f64<float>(float v) { return (double)v; }
template <> __device__ __forceinline__ double to_f64<double>(double v) { return v; }
template <> __device__ __forceinline__ double to_f64<uint16_t>(uint16_t v) { return (double)bf16_to_f32(v); }

__device__ __forceinline__ int block_reduce_int(int v, int* red, bool take_max) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const int t = __shfl_xor_sync(0xffffffffu, v, o);
        v = take_max ? max(v, t) : min(v, t);
    }
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        int t = lane < nw ? red[lane] : (take_max ? INT_MIN : INT_MAX);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const int u = __shfl_xor_sync(0xffffffffu, t, o);
            t = take_max ? max(t, u) : min(t, u);
        }
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ w, int K, uint32_t* __restrict__ codes,
                                                       uint8_t* __restrict__ bcodes, float* __restrict__ wscale,
                                                       int8_t* __restrict__ qw, int32_t* __restrict__ row_exp) {
    extern __shared__ int s_e[];          // per-block exponent of this row (INT_MIN = all-zero block)
    __shared__ int red[33];
    const int64_t n = blockIdx.x;
    const int nb = K / 32;
    const T* wr = w + n * (int64_t)K;

    int hi = INT_MIN;
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        double v[32];
        double amax = 0.0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            v[i] = to_f64<T>(wr[b * 32 + i]);
            amax = fmax(amax, fabs(v[i]));
        }
        int e;
        if (amax == 0.0) {
            e = INT_MIN;
        } else {
            const int e0 = ilogb(amax) - 2;
            int best = e0;
            double err = block_sq_err(v, e0);
            const double em = block_sq_err(v, e0 - 1);
            if (em < err) { best = e0 - 1; err = em; }
            const double ep = block_sq_err(v, e0 + 1);
            if (ep < err) { best = e0 + 1; err = ep; }
            e = best;
        }
        s_e[b] = e;
        hi = max(hi, e);
    }
    hi = block_reduce_int(hi, red, true);
    if (hi == INT_MIN) hi = 0;            // all-zero row
    const int lo_c = hi - 3;
    int lo = INT_MAX;
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        const int e = max(s_e[b], lo_c);
        s_e[b] = e;
        lo = min(lo, e);
    }
    lo = block_reduce_int(lo, red, false);   // E_lo (also syncs s_e)
    if (threadIdx.x == 0) {
        wscale[n] = (float)scalbn(1.0, lo - 1);
        if (row_exp) row_exp[n] = lo;
    }
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        const int e = s_e[b];
        const int shift = e - lo;
        const double si = scalbn(1.0, -e);
        uint32_t words[4];
        uint32_t qwords[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const double t = __dmul_rn(to_f64<T>(wr[b * 32 + 8 * j + i]), si);
                const int idx = e2m1_idx(fabs(t));
                const int neg = (t < 0.0) && idx > 0;
                word |= (uint32_t)(idx | (neg << 3)) << (4 * i);
                const int q = e2m1_x2(idx) << shift;
                const uint32_t qb = (uint32_t)(neg ? -q : q) & 0xFFu;
                if (i < 4) qwords[2 * j] = (i == 0 ? 0u : qwords[2 * j]) | (qb << (8 * i));
                else qwords[2 * j + 1] = (i == 4 ? 0u : qwords[2 * j + 1]) | (qb << (8 * (i - 4)));
            }
            words[j] = word;
        }
        reinterpret_cast<uint4*>(codes + n * (int64_t)(K / 8))[b] = make_uint4(words[0], words[1], words[2], words[3]);
        if (qw) {
            uint4* q4 = reinterpret_cast<uint4*>(qw + n * (int64_t)K + b * 32);
            q4[0] = make_uint4(qwords[0], qwords[1], qwords[2], qwords[3]);
            q4[1] = make_uint4(qwords[4], qwords[5], qwords[6], qwords[7]);
        }
        if ((b & 3) == 0) {
            const uint32_t byte = (uint32_t)(s_e[b] - lo) | ((uint32_t)(s_e[b + 1] - lo) << 2) |
                                  ((uint32_t)(s_e[b + 2] - lo) << 4) | ((uint32_t)(s_e[b + 3] - lo) << 6);
            bcodes[n * (int64_t)(nb / 4) + b / 4] = (uint8_t)byte;
        }
    }
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_quantize_sc_mxfp4(const void* w, int w_dtype, int64_t N, int64_t K, uint32_t* codes, uint8_t* bcodes,
                                      float* wscale, int8_t* qw, int32_t* row_exp, void* stream) {
    SCMX_REQUIRE(N >= 0 && K > 0 && K % 128 == 0 && K <= (1 << 20), SCMX_EINVAL,
                 "quantize_sc_mxfp4: K=%lld must be a positive multiple of 128", (long long)K);
    SCMX_REQUIRE(w_dtype >= 0 && w_dtype <= 2, SCMX_EINVAL, "quantize_sc_mxfp4: w_dtype=%d (0 f32, 1 f64, 2 bf16)", w_dtype);
    SCMX_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 15) == 0 && (!qw || (reinterpret_cast<uintptr_t>(qw) & 15) == 0),
                 SCMX_EINVAL, "quantize_sc_mxfp4: codes and qw must be 16-byte aligned");
    if (N == 0) return SCMX_OK;
    const int nb = (int)(K / 32);
    int threads = nb < 256 ? ((nb + 31) / 32) * 32 : 256;
    const size_t smem = (size_t)nb * sizeof(int);
    cudaStream_t st = (cudaStream_t)stream;
    if (w_dtype == 0)
        quantize_kernel<float><<<(unsigned)N, threads, smem, st>>>((const float*)w, (int)K, codes, bcodes, wscale, qw, row_exp);
    else if (w_dtype == 1)
        quantize_kernel<double><<<(unsigned)N, threads, smem, st>>>((const double*)w, (int)K, codes, bcodes, wscale, qw, row_exp);
    else
        quantize_kernel<uint16_t><<<(unsigned)N, threads, smem, st>>>((const uint16_t*)w, (int)K, codes, bcodes, wscale, qw, row_exp);
    SCMX_LAUNCH_OK("quantize_kernel");
    return SCMX_OK;
}
