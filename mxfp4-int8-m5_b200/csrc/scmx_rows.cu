// HBM-bound row kernels of the W4A8 path: weight unpack, per-token INT8 activation quantization, RMSNorm + quant,
// residual / SwiGLU epilogues on INT32 accumulators, MoE combine, row gather.  One CTA per activation row;
// 128-bit loads; reductions by warp shuffle + shared memory.
#include "scmx_common.cuh"

namespace scmx {

// ---- unpack: thread = one uint4 of codes (32 weights); block = 64 vectors x 4 rows, no index divisions ---------------------
__global__ void __launch_bounds__(256) unpack_kernel(const uint4* __restrict__ codes, const uint8_t* __restrict__ bcodes,
                                                     int64_t N, int vec_per_row, int bc_row_bytes, DevFormat f,
                                                     uint4* __restrict__ wq) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t n = (int64_t)blockIdx.x * 4 + threadIdx.y;
    const int v = blockIdx.y * 64 + threadIdx.x;
    if (n >= N || v >= vec_per_row) return;
    const int64_t i = n * vec_per_row + v;
    const int k0 = v * 32;
    const uint4 c = codes[i];
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
    const uint8_t* bc = bcodes + n * bc_row_bytes;
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t m = fmt_mult(f, block_code_fast(f, bc, block_of(f, k0 + 8 * j)));
        const uint32_t plo = lut_scale(f.mag_lo, m), phi = lut_scale(f.mag_hi, m);
        decode_word(w[j], plo, phi, lut_negate(plo), lut_negate(phi), o[2 * j], o[2 * j + 1]);
    }
    wq[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    wq[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// ---- helpers: a row of K values processed by the CTA in vectors of 8 --------------------------------------------
__device__ __forceinline__ void load8_bf16(const uint16_t* p, float v[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ void store8_i8(int8_t* p, const int q[8]) {
    uint2 o;
    o.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    o.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
    *reinterpret_cast<uint2*>(p) = o;
}
__device__ __forceinline__ void store8_bf16(uint16_t* p, const float v[8]) {
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]);
    o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = o;
}

// Eight elements of a row normalized in place: f[j] = T(w[j] * T(f[j] * inv)), T = round to bfloat16; returns them packed.
// Roundings are taken two at a time (pack_bf16x2).
__device__ __forceinline__ uint4 norm8(float (&f)[8], const uint4& wraw, float inv) {
    const uint32_t w[4] = {wraw.x, wraw.y, wraw.z, wraw.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t t = pack_bf16x2(__fmul_rn(f[2 * j], inv), __fmul_rn(f[2 * j + 1], inv));
        o[j] = pack_bf16x2(__fmul_rn(bf16_lo(w[j]), bf16_lo(t)), __fmul_rn(bf16_hi(w[j]), bf16_hi(t)));
        f[2 * j] = bf16_lo(o[j]);
        f[2 * j + 1] = bf16_hi(o[j]);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// ---- act_quant -------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) act_quant_kernel(const uint16_t* __restrict__ x, int64_t M, int K,
                                                        int8_t* __restrict__ xq, float* __restrict__ xs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int64_t row = blockIdx.x;
    int8_t* qrow = xq + row * K;
    if (row >= M) {   // padded rows: zero codes, zero scale
        for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) *reinterpret_cast<uint2*>(qrow + k) = make_uint2(0, 0);
        if (threadIdx.x == 0) xs[row] = 0.0f;
        return;
    }
    const uint16_t* xrow = x + row * K;
    float amax = 0.0f;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        load8_bf16(xrow + k, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        int q[8];
        load8_bf16(xrow + k, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = quant_code(v[j], qi);
        store8_i8(qrow + k, q);
    }
    if (threadIdx.x == 0) xs[row] = s;
}

// ---- RMSNorm + quant (optionally writing the normalized bf16 row) -----------------------------------------------
// inv = 1 / sqrt(float(sum x^2) / K + eps): the sum of squares is accumulated in float64 (exact for bf16 inputs of
// ordinary dynamic range, hence independent of the reduction order), the reciprocal square root in float64.

__global__ void __launch_bounds__(256) rmsnorm_quant_kernel(const uint16_t* __restrict__ x,
                                                            const uint16_t* __restrict__ nw, float eps, int64_t M, int K,
                                                            int8_t* __restrict__ xq, float* __restrict__ xs,
                                                            uint16_t* __restrict__ xn) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    __shared__ double dred[33];
    const int64_t row = blockIdx.x;
    int8_t* qrow = xq + row * K;
    if (row >= M) {
        for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
            *reinterpret_cast<uint2*>(qrow + k) = make_uint2(0, 0);
            if (xn) *reinterpret_cast<uint4*>(xn + row * K + k) = make_uint4(0, 0, 0, 0);
        }
        if (threadIdx.x == 0) xs[row] = 0.0f;
        return;
    }
    const uint16_t* xrow = x + row * K;
    double ss = 0.0;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        load8_bf16(xrow + k, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += sq_f64(v[j]);
    }
    ss = block_sum(ss, dred);
    const float inv = rms_inverse(ss, K, eps);
    float amax = 0.0f;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        load8_bf16(xrow + k, v);
        const uint4 o = norm8(v, *reinterpret_cast<const uint4*>(nw + k), inv);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        if (xn) *reinterpret_cast<uint4*>(xn + row * K + k) = o;
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        int q[8];
        load8_bf16(xrow + k, v);
        norm8(v, *reinterpret_cast<const uint4*>(nw + k), inv);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = quant_code(v[j], qi);
        store8_i8(qrow + k, q);
    }
    if (threadIdx.x == 0) xs[row] = s;
}

// Input rows may be stored in column segments (the layout an all-gather of column shards produces): element
// (m, s * w + j) lives at x[s * seg_stride + m * w + j].  One segment of width K is the ordinary row-major matrix.
struct RowSegs {
    int w8;              // 16-byte vectors per segment row
    int64_t stride8;     // distance between segments in 16-byte vectors
    // position of 16-byte vector v of row `row`; ordinary matrices (one segment) need no division
    __device__ __forceinline__ int64_t index(int64_t row, int v) const {
        if (stride8 == 0) return row * w8 + v;
        return (int64_t)(v / w8) * stride8 + row * w8 + (v % w8);
    }
};

// ---- warp-per-row variants (K <= 256 * MAXV): the whole row lives in registers, reductions are shuffles only -------------
__device__ __forceinline__ void unpack8(const uint4& r, float v[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint2 pack8_i8(const int q[8]) {
    uint2 o;
    o.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    o.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
    return o;
}

// WPR warps share a row (WPR = 1, 2 or 4; 8 / WPR rows per CTA): each lane holds MAXV vectors, vector v = (i * WPR + part) * 32 +
// lane.  With few rows (one warp per row leaves an SM a dozen warps) splitting a row shortens every warp's dependent chain and
// doubles the warps that hide it; the partial sums and maxima meet through shared memory behind a barrier of the row's warps.
template <int MAXV, bool NORM, int WPR>
__global__ void __launch_bounds__(256) row_quant_warp_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ nw,
                                                             float eps, int64_t M, int64_t Mp, int K, RowSegs sg,
                                                             int8_t* __restrict__ xq, float* __restrict__ xs,
                                                             uint16_t* __restrict__ xn) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ double s_ss[8];
    __shared__ float s_am[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rin = warp / WPR, part = warp % WPR;          // row inside the CTA, this warp's part of it
    const int64_t row = (int64_t)blockIdx.x * (8 / WPR) + rin;
    if (row >= Mp) return;                                    // all warps of a row leave together
    const int nv = K / 8;                      // 16-byte vectors per row
    uint2* qrow = reinterpret_cast<uint2*>(xq + row * K);
    if (row >= M) {                            // padded rows: zero codes, zero scale
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int v = (i * WPR + part) * 32 + lane;
            if (v < nv) {
                qrow[v] = make_uint2(0, 0);
                if (NORM && xn) reinterpret_cast<uint4*>(xn + row * K)[v] = make_uint4(0, 0, 0, 0);
            }
        }
        if (lane == 0 && part == 0) xs[row] = 0.0f;
        return;
    }
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    uint4 raw[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = (i * WPR + part) * 32 + lane;
        raw[i] = v < nv ? x4[sg.index(row, v)] : make_uint4(0, 0, 0, 0);
    }
    float inv = 1.0f;
    if (NORM) {
        double s4[4] = {0.0, 0.0, 0.0, 0.0};      // four chains instead of one: every partial sum is exact, so the grouping is free
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            float f[8];
            unpack8(raw[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) s4[j & 3] += sq_f64(f[j]);
        }
        double ss = (s4[0] + s4[1]) + (s4[2] + s4[3]);
        ss = warp_sum(ss);
        if (WPR > 1) {
            if (lane == 0) s_ss[warp] = ss;
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rin), "n"(32 * WPR) : "memory");
            ss = 0.0;
#pragma unroll
            for (int p = 0; p < WPR; ++p) ss += s_ss[rin * WPR + p];
        }
        inv = rms_inverse(ss, K, eps);
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = (i * WPR + part) * 32 + lane;
        float f[8];
        unpack8(raw[i], f);
        if (NORM && v < nv) {
            const uint4 o = norm8(f, reinterpret_cast<const uint4*>(nw)[v], inv);
            raw[i] = o;                        // keep the normalized row (bf16) for the quantization pass
            if (xn) reinterpret_cast<uint4*>(xn + row * K)[v] = o;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    }
    amax = warp_max(amax);
    if (WPR > 1) {
        if (lane == 0) s_am[warp] = amax;
        asm volatile("bar.sync %0, %1;" ::"r"(1 + rin), "n"(32 * WPR) : "memory");
        amax = 0.0f;
#pragma unroll
        for (int p = 0; p < WPR; ++p) amax = fmaxf(amax, s_am[rin * WPR + p]);
    }
    float s, qi;
    quant_scale(amax, s, qi);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = (i * WPR + part) * 32 + lane;
        if (v < nv) {
            float f[8];
            unpack8(raw[i], f);
            qrow[v] = make_uint2(quant4(f[0], f[1], f[2], f[3], qi), quant4(f[4], f[5], f[6], f[7], qi));
        }
    }
    if (lane == 0 && part == 0) xs[row] = s;
}

// CTA-per-row variant for wider rows (K <= 2048 * MAXV): each thread keeps MAXV 16-byte vectors of the row in registers.
template <int MAXV, bool NORM>
__global__ void __launch_bounds__(256) row_quant_block_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ nw,
                                                              float eps, int64_t M, int K, RowSegs sg, int8_t* __restrict__ xq,
                                                              float* __restrict__ xs, uint16_t* __restrict__ xn) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    __shared__ double dred[33];
    const int64_t row = blockIdx.x;
    const int nv = K / 8;
    uint2* qrow = reinterpret_cast<uint2*>(xq + row * K);
    if (row >= M) {
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int v = i * 256 + threadIdx.x;
            if (v < nv) {
                qrow[v] = make_uint2(0, 0);
                if (NORM && xn) reinterpret_cast<uint4*>(xn + row * K)[v] = make_uint4(0, 0, 0, 0);
            }
        }
        if (threadIdx.x == 0) xs[row] = 0.0f;
        return;
    }
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    uint4 raw[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = i * 256 + threadIdx.x;
        raw[i] = v < nv ? x4[sg.index(row, v)] : make_uint4(0, 0, 0, 0);
    }
    float inv = 1.0f;
    if (NORM) {
        double s4[4] = {0.0, 0.0, 0.0, 0.0};      // four chains instead of one: every partial sum is exact, so the grouping is free
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            float f[8];
            unpack8(raw[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) s4[j & 3] += sq_f64(f[j]);
        }
        double ss = (s4[0] + s4[1]) + (s4[2] + s4[3]);
        ss = block_sum(ss, dred);
        inv = rms_inverse(ss, K, eps);
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = i * 256 + threadIdx.x;
        float f[8];
        unpack8(raw[i], f);
        if (NORM && v < nv) {
            const uint4 o = norm8(f, reinterpret_cast<const uint4*>(nw)[v], inv);
            raw[i] = o;
            if (xn) reinterpret_cast<uint4*>(xn + row * K)[v] = o;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = i * 256 + threadIdx.x;
        if (v < nv) {
            float f[8];
            unpack8(raw[i], f);
            qrow[v] = make_uint2(quant4(f[0], f[1], f[2], f[3], qi), quant4(f[4], f[5], f[6], f[7], qi));
        }
    }
    if (threadIdx.x == 0) xs[row] = s;
}

template <bool NORM>
static bool launch_row_quant_warp(const uint16_t* x, const uint16_t* nw, float eps, int64_t M, int64_t Mp, int64_t K,
                                  int nseg, int64_t seg_stride, int8_t* xq, float* xs, uint16_t* xn, cudaStream_t st) {
    const unsigned grid = (unsigned)((Mp + 7) / 8);
    RowSegs sg;
    sg.w8 = (int)(K / nseg / 8);
    sg.stride8 = seg_stride / 8;
    // a handful of rows (decode): one CTA per row keeps the dependent chain short; many rows: one warp per row
    // (measured: at 2048+ rows the warp-per-row kernels are as fast or faster: 8.2 vs 8.6 us RMSNorm+INT8 at 2048 x 2048,
    // 16 vs 42 us act-quant at 32768 x 1024)
    constexpr int64_t block_rows = 32;
    // a few thousand rows of 1024 - 2048 elements: several warps per row.  Measured inside the dense step at M = 2048 (the
    // kernel alone, launched back to back, prefers one warp per row): RMSNorm + INT8 with 4 warps per row 3.754 -> 3.705 ms per
    // step, act-quant with 2 warps per row a further 0.008 ms.
    const int wpr = (Mp <= 4096 && K > 1024 && K <= 2048) ? (NORM ? 4 : 2) : 1;     // 8 / 4 warps per row measured slower: 3.70 - 3.73 ms
    if (Mp <= block_rows && K <= 2048) launch_pdl(row_quant_block_kernel<1, NORM>, dim3((unsigned)Mp), dim3(256), 0, st, x, nw, eps, M, (int)K, sg, xq, xs, xn);
    else if (Mp <= block_rows && K <= 2048 * 4) launch_pdl(row_quant_block_kernel<4, NORM>, dim3((unsigned)Mp), dim3(256), 0, st, x, nw, eps, M, (int)K, sg, xq, xs, xn);
    else if (wpr == 2 && K <= 256 * 8) launch_pdl(row_quant_warp_kernel<4, NORM, 2>, dim3((unsigned)((Mp + 3) / 4)), dim3(256), 0, st, x, nw, eps, M, Mp, (int)K, sg, xq, xs, xn);
    else if (wpr == 4 && K <= 256 * 8) launch_pdl(row_quant_warp_kernel<2, NORM, 4>, dim3((unsigned)((Mp + 1) / 2)), dim3(256), 0, st, x, nw, eps, M, Mp, (int)K, sg, xq, xs, xn);
    else if (K <= 256 * 4) launch_pdl(row_quant_warp_kernel<4, NORM, 1>, dim3(grid), dim3(256), 0, st, x, nw, eps, M, Mp, (int)K, sg, xq, xs, xn);
    else if (K <= 256 * 8) launch_pdl(row_quant_warp_kernel<8, NORM, 1>, dim3(grid), dim3(256), 0, st, x, nw, eps, M, Mp, (int)K, sg, xq, xs, xn);
    else if (K <= 256 * 16) launch_pdl(row_quant_warp_kernel<16, NORM, 1>, dim3(grid), dim3(256), 0, st, x, nw, eps, M, Mp, (int)K, sg, xq, xs, xn);
    else if (K <= 2048 * 4) launch_pdl(row_quant_block_kernel<4, NORM>, dim3((unsigned)Mp), dim3(256), 0, st, x, nw, eps, M, (int)K, sg, xq, xs, xn);
    else return false;
    return true;
}

// ---- residual epilogue on INT32 accumulators ---------------------------------------------------------------------
__global__ void __launch_bounds__(256) res_epilogue_kernel(const int32_t* __restrict__ acc, const float* __restrict__ xscale,
                                                           const float* __restrict__ wscale,
                                                           const uint16_t* __restrict__ res, int64_t total4, int N,
                                                           uint16_t* __restrict__ h) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int64_t e = i * 4;
    const int64_t m = e / N;
    const int n = (int)(e % N);
    const int4 a = *reinterpret_cast<const int4*>(acc + e);
    const float4 ws = *reinterpret_cast<const float4*>(wscale + n);
    const uint2 r = *reinterpret_cast<const uint2*>(res + e);
    const float xsm = xscale[m];
    const float y0 = rbf(__fadd_rn(__uint_as_float(r.x << 16), scale_acc(a.x, xsm, ws.x)));
    const float y1 = rbf(__fadd_rn(__uint_as_float(r.x & 0xFFFF0000u), scale_acc(a.y, xsm, ws.y)));
    const float y2 = rbf(__fadd_rn(__uint_as_float(r.y << 16), scale_acc(a.z, xsm, ws.z)));
    const float y3 = rbf(__fadd_rn(__uint_as_float(r.y & 0xFFFF0000u), scale_acc(a.w, xsm, ws.w)));
    uint2 o;
    o.x = f32_to_bf16(y0) | ((uint32_t)f32_to_bf16(y1) << 16);
    o.y = f32_to_bf16(y2) | ((uint32_t)f32_to_bf16(y3) << 16);
    *reinterpret_cast<uint2*>(h + e) = o;
}

// ---- SwiGLU of gate | up accumulators, then per-token INT8 ----------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_quant_kernel(const int32_t* __restrict__ acc, const float* __restrict__ xscale,
                                                           const float* __restrict__ wscale, int F, int8_t* __restrict__ xq,
                                                           float* __restrict__ xs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int64_t row = blockIdx.x;
    const int32_t* ar = acc + row * 2 * (int64_t)F;
    const float xsr = xscale[row];
    float amax = 0.0f;
    for (int c = threadIdx.x * 4; c < F; c += blockDim.x * 4) {
        const int4 g4 = *reinterpret_cast<const int4*>(ar + c);
        const int4 u4 = *reinterpret_cast<const int4*>(ar + F + c);
        const float4 wg = *reinterpret_cast<const float4*>(wscale + c);
        const float4 wu = *reinterpret_cast<const float4*>(wscale + F + c);
        amax = fmaxf(amax, fabsf(swiglu_bf16(scale_acc(g4.x, xsr, wg.x), scale_acc(u4.x, xsr, wu.x))));
        amax = fmaxf(amax, fabsf(swiglu_bf16(scale_acc(g4.y, xsr, wg.y), scale_acc(u4.y, xsr, wu.y))));
        amax = fmaxf(amax, fabsf(swiglu_bf16(scale_acc(g4.z, xsr, wg.z), scale_acc(u4.z, xsr, wu.z))));
        amax = fmaxf(amax, fabsf(swiglu_bf16(scale_acc(g4.w, xsr, wg.w), scale_acc(u4.w, xsr, wu.w))));
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
    for (int c = threadIdx.x * 4; c < F; c += blockDim.x * 4) {
        const int4 g4 = *reinterpret_cast<const int4*>(ar + c);
        const int4 u4 = *reinterpret_cast<const int4*>(ar + F + c);
        const float4 wg = *reinterpret_cast<const float4*>(wscale + c);
        const float4 wu = *reinterpret_cast<const float4*>(wscale + F + c);
        const int q0 = quant_code(swiglu_bf16(scale_acc(g4.x, xsr, wg.x), scale_acc(u4.x, xsr, wu.x)), qi);
        const int q1 = quant_code(swiglu_bf16(scale_acc(g4.y, xsr, wg.y), scale_acc(u4.y, xsr, wu.y)), qi);
        const int q2 = quant_code(swiglu_bf16(scale_acc(g4.z, xsr, wg.z), scale_acc(u4.z, xsr, wu.z)), qi);
        const int q3 = quant_code(swiglu_bf16(scale_acc(g4.w, xsr, wg.w), scale_acc(u4.w, xsr, wu.w)), qi);
        *reinterpret_cast<uint32_t*>(xq + row * F + c) =
            (q0 & 0xFF) | ((q1 & 0xFF) << 8) | ((q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    }
    if (threadIdx.x == 0) xs[row] = s;
}

__global__ void swiglu_kernel(const uint16_t* __restrict__ g, const uint16_t* __restrict__ u, int64_t n,
                              uint16_t* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_bf16(swiglu_bf16(bf16_to_f32(g[i]), bf16_to_f32(u[i])));
}

// ---- MoE combine ------------------------------------------------------------------------------------------------------
// acc_j = rbf(rbf(y[pos[t*k+j]] * sc_j) + acc_{j-1}), h = T(res + acc); then (QUANT) RMSNorm + INT8 of h.
// Expert-parallel "pull" form: the expert outputs stay on the GPUs that computed them, stored by receive slot
// [source rank * cap + position among the rows that source sent]; the combine of the GPU that owns the token reads them
// over peer memory.  Sorted position p of this rank went to rank d = es[p] / El at slot rank * cap + (p - off[d * El]).
struct CombinePull {
    const int32_t* es;            // expert of every sorted position; null = local form (rows of y at pos)
    const int32_t* off;           // this rank's segment offsets per global expert
    const uint16_t* peer[8];      // every rank's slot-ordered output buffer
    int El, cap, rank, world;
};

// Four CTAs per SM (63 registers): the kernel is a chain index loads -> barrier -> row loads -> sum -> store per CTA, hidden
// only by other resident CTAs; with three per SM (67 registers) it ran at 42 % of DRAM throughput, 45 us against 39 us now
// for 4096 tokens x 8 experts x 2048.
template <int TOPK_MAX>
__global__ void __launch_bounds__(256, 4) moe_combine_kernel(const uint16_t* __restrict__ y, const int32_t* __restrict__ pos,
                                                          const uint16_t* __restrict__ scores,
                                                          const uint16_t* __restrict__ res, const uint16_t* __restrict__ nw,
                                                          float eps, int64_t M, int K, int topk, int quant,
                                                          uint16_t* __restrict__ h, int8_t* __restrict__ xq,
                                                          float* __restrict__ xs, const CombinePull pl) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    __shared__ double dred[33];
    __shared__ const uint16_t* s_ptr[TOPK_MAX];
    __shared__ float s_sc[TOPK_MAX];
    const int64_t row = blockIdx.x;
    const bool live = row < M;
    if (live && threadIdx.x < topk) {
        const int p = pos[row * topk + threadIdx.x];
        const uint16_t* base = y + (int64_t)p * K;
        if (pl.es != nullptr) {
            const int e = pl.es[p];
            const int d = e / pl.El;
            const int idx = (d >= 0 && d < pl.world) ? p - pl.off[d * pl.El] : -1;
            // inconsistent routing tables: contribute zeros instead of reading somewhere
            base = (idx >= 0 && idx < pl.cap && pl.peer[d] != nullptr) ? pl.peer[d] + ((int64_t)pl.rank * pl.cap + idx) * K : nullptr;
        }
        s_ptr[threadIdx.x] = base;
        s_sc[threadIdx.x] = bf16_to_f32(scores[row * topk + threadIdx.x]);
    }
    __syncthreads();
    const uint16_t* rrow = res + row * K;
    uint16_t* hrow = h + row * K;
    double ss = 0.0;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float r[8], a[8];
        load8_bf16(rrow + k, r);
        if (live) {
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = 0.0f;
            for (int t0 = 0; t0 < topk; t0 += 8) {            // up to 8 expert rows in flight, summed in slot order
                uint4 raw[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (t0 + u < topk)
                        raw[u] = s_ptr[t0 + u] ? *reinterpret_cast<const uint4*>(s_ptr[t0 + u] + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (t0 + u < topk) {
                        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                        const float sc = s_sc[t0 + u];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {           // roundings two at a time
                            const uint32_t t = pack_bf16x2(__fmul_rn(bf16_lo(w[j]), sc), __fmul_rn(bf16_hi(w[j]), sc));
                            const uint32_t s2 = pack_bf16x2(__fadd_rn(bf16_lo(t), a[2 * j]), __fadd_rn(bf16_hi(t), a[2 * j + 1]));
                            a[2 * j] = bf16_lo(s2);
                            a[2 * j + 1] = bf16_hi(s2);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t s2 = pack_bf16x2(__fadd_rn(r[2 * j], a[2 * j]), __fadd_rn(r[2 * j + 1], a[2 * j + 1]));
                r[2 * j] = bf16_lo(s2);
                r[2 * j + 1] = bf16_hi(s2);
            }
        }
        store8_bf16(hrow + k, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += sq_f64(r[j]);
    }
    if (!quant) return;
    int8_t* qrow = xq + row * K;
    __syncthreads();   // h row written by this CTA is re-read below
    ss = block_sum(ss, dred);
    const float inv = rms_inverse(ss, K, eps);
    float amax = 0.0f;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        load8_bf16(hrow + k, v);
        norm8(v, *reinterpret_cast<const uint4*>(nw + k), inv);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        int q[8];
        load8_bf16(hrow + k, v);
        norm8(v, *reinterpret_cast<const uint4*>(nw + k), inv);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = quant_code(v[j], qi);
        store8_i8(qrow + k, q);
    }
    if (threadIdx.x == 0) xs[row] = s;
}

// ---- row gather --------------------------------------------------------------------------------------------------------
// One warp per destination row: its 16-byte loads are all issued before the first store (K <= 8192: 16 per lane).
__global__ void __launch_bounds__(256) gather_rows_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs,
                                                          const int32_t* __restrict__ tok, int64_t rows_q, int64_t rows_s, int K,
                                                          int8_t* __restrict__ dq, float* __restrict__ ds) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (p >= rows_q) return;
    const int t = tok[p];
    const uint4* src = reinterpret_cast<const uint4*>(xq + (int64_t)t * K);
    uint4* dst = reinterpret_cast<uint4*>(dq + p * K);
    const int nv = K / 16;
    for (int base = 0; base < nv; base += 32 * 8) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * 32 + lane;
            if (i < nv) v[j] = src[i];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = base + j * 32 + lane;
            if (i < nv) dst[i] = v[j];
        }
    }
    if (lane == 0 && p < rows_s) ds[p] = xs[t];
}

// ---- rotated-input quantization --------------------------------------------------------------------------------------------
// Every 32-wide block of the row is multiplied by a +-1 sign vector and by the 32-point Hadamard matrix, scaled by 1/sqrt(32),
// rounded to bf16, then the row is quantized per token like act_quant.  The float32 butterflies run in the order of
// e2e/sc_kernels.py:234-275 (two stages inside a thread's 4 values, three across the 8 threads of a block: the thread whose
// index has bit h set computes partner - own, the other own + partner), so the sums round identically.
constexpr float ROT_NORM = 0.17677669529663687f;

__global__ void __launch_bounds__(256) rot_quant_kernel(const uint16_t* __restrict__ x, const float* __restrict__ signs, int64_t M,
                                                        int K, int8_t* __restrict__ xq, float* __restrict__ xs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    constexpr int MAXJ = 8;                                   // K <= 8192
    const int64_t row = blockIdx.x;
    const int t = threadIdx.x;
    float v[MAXJ][4];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
        const int p = 4 * (j * 256 + t);
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        if (p < K && row < M) {
            const uint2 r = *reinterpret_cast<const uint2*>(x + row * K + p);
            const float4 sg = *reinterpret_cast<const float4*>(signs + p);
            a0 = __fmul_rn(__uint_as_float(r.x << 16), sg.x);
            a1 = __fmul_rn(__uint_as_float(r.x & 0xFFFF0000u), sg.y);
            a2 = __fmul_rn(__uint_as_float(r.y << 16), sg.z);
            a3 = __fmul_rn(__uint_as_float(r.y & 0xFFFF0000u), sg.w);
        }
        float b0 = __fadd_rn(a0, a1), b1 = __fsub_rn(a0, a1), b2 = __fadd_rn(a2, a3), b3 = __fsub_rn(a2, a3);
        a0 = __fadd_rn(b0, b2); a1 = __fadd_rn(b1, b3); a2 = __fsub_rn(b0, b2); a3 = __fsub_rn(b1, b3);
#pragma unroll
        for (int h = 1; h < 8; h <<= 1) {                     // every lane takes part: the trip count is uniform
            const float c0 = __shfl_xor_sync(0xffffffffu, a0, h), c1 = __shfl_xor_sync(0xffffffffu, a1, h);
            const float c2 = __shfl_xor_sync(0xffffffffu, a2, h), c3 = __shfl_xor_sync(0xffffffffu, a3, h);
            if (t & h) {
                a0 = __fsub_rn(c0, a0); a1 = __fsub_rn(c1, a1); a2 = __fsub_rn(c2, a2); a3 = __fsub_rn(c3, a3);
            } else {
                a0 = __fadd_rn(a0, c0); a1 = __fadd_rn(a1, c1); a2 = __fadd_rn(a2, c2); a3 = __fadd_rn(a3, c3);
            }
        }
        v[j][0] = rbf(__fmul_rn(a0, ROT_NORM)); v[j][1] = rbf(__fmul_rn(a1, ROT_NORM));
        v[j][2] = rbf(__fmul_rn(a2, ROT_NORM)); v[j][3] = rbf(__fmul_rn(a3, ROT_NORM));
#pragma unroll
        for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
        const int p = 4 * (j * 256 + t);
        if (p < K) *reinterpret_cast<uint32_t*>(xq + row * K + p) = quant4(v[j][0], v[j][1], v[j][2], v[j][3], qi);
    }
    if (t == 0) xs[row] = s;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_unpack_i8(const uint32_t* codes, const uint8_t* bcodes, int64_t N, int64_t K, const scmx_format* fmt,
                              int8_t* wq, void* stream) {
    DevFormat f;
    int rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    SCMX_REQUIRE(N >= 0 && K > 0 && K % 32 == 0 && K % (f.block * f.blocks_per_byte) == 0, SCMX_EINVAL,
                 "unpack_i8: K=%lld must be a multiple of 32 and of block*codes_per_byte=%d", (long long)K,
                 f.block * f.blocks_per_byte);
    SCMX_REQUIRE(f.block % 8 == 0 && (32 % f.block == 0 || f.block % 32 == 0), SCMX_EFORMAT,
                 "unpack_i8: block=%d must divide or be a multiple of 32", f.block);
    SCMX_REQUIRE(aligned16(codes) && aligned16(wq), SCMX_EINVAL, "unpack_i8: codes and wq must be 16-byte aligned");
    if (N == 0) return SCMX_OK;
    const int vec_per_row = (int)(K / 32);
    const int bc_row = (int)(K / (f.block * f.blocks_per_byte));
    SCMX_REQUIRE((vec_per_row + 63) / 64 <= 65535, SCMX_ELIMIT, "unpack_i8: K too large");
    launch_pdl(unpack_kernel, dim3((unsigned)((N + 3) / 4), (unsigned)((vec_per_row + 63) / 64)), dim3(64, 4), 0,
               (cudaStream_t)stream, reinterpret_cast<const uint4*>(codes), bcodes, N, vec_per_row, bc_row, f,
               reinterpret_cast<uint4*>(wq));
    SCMX_LAUNCH_OK("unpack_kernel");
    return SCMX_OK;
}

extern "C" int scmx_act_quant(const uint16_t* x, int64_t M, int64_t K, int64_t Mp, int8_t* xq, float* xs, void* stream) {
    SCMX_REQUIRE(M >= 0 && Mp >= M && K > 0 && K % 8 == 0 && K <= (1 << 20), SCMX_EINVAL,
                 "act_quant: need 0 <= M <= Mp and K %% 8 == 0 (M=%lld Mp=%lld K=%lld)", (long long)M, (long long)Mp,
                 (long long)K);
    SCMX_REQUIRE(aligned16(x) && aligned16(xq) && K % 8 == 0, SCMX_EINVAL, "act_quant: x and xq must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    if (!launch_row_quant_warp<false>(x, nullptr, 0.0f, M, Mp, K, 1, 0, xq, xs, nullptr, (cudaStream_t)stream))
        launch_pdl(act_quant_kernel, dim3((unsigned)Mp), dim3(256), 0, (cudaStream_t)stream, x, M, (int)K, xq, xs);
    SCMX_LAUNCH_OK("act_quant_kernel");
    return SCMX_OK;
}

extern "C" int scmx_rmsnorm_quant(const uint16_t* x, const uint16_t* nw, float eps, int64_t M, int64_t K, int64_t Mp,
                                  int8_t* xq, float* xs, uint16_t* xn, void* stream) {
    SCMX_REQUIRE(M >= 0 && Mp >= M && K > 0 && K % 8 == 0 && K <= (1 << 20), SCMX_EINVAL,
                 "rmsnorm_quant: need 0 <= M <= Mp and K %% 8 == 0 (M=%lld Mp=%lld K=%lld)", (long long)M,
                 (long long)Mp, (long long)K);
    SCMX_REQUIRE(aligned16(x) && aligned16(nw) && aligned16(xq) && (!xn || aligned16(xn)), SCMX_EINVAL,
                 "rmsnorm_quant: buffers must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    if (!launch_row_quant_warp<true>(x, nw, eps, M, Mp, K, 1, 0, xq, xs, xn, (cudaStream_t)stream))
        launch_pdl(rmsnorm_quant_kernel, dim3((unsigned)Mp), dim3(256), 0, (cudaStream_t)stream, x, nw, eps, M, (int)K, xq, xs, xn);
    SCMX_LAUNCH_OK("rmsnorm_quant_kernel");
    return SCMX_OK;
}

extern "C" int scmx_res_epilogue(const int32_t* acc, const float* xscale, const float* wscale, const uint16_t* res,
                                 int64_t Mp, int64_t N, uint16_t* h, void* stream) {
    SCMX_REQUIRE(Mp >= 0 && N > 0 && N % 4 == 0, SCMX_EINVAL, "res_epilogue: N=%lld must be a multiple of 4", (long long)N);
    SCMX_REQUIRE(aligned16(acc) && aligned16(wscale) && aligned16(res) && aligned16(h), SCMX_EINVAL,
                 "res_epilogue: buffers must be 16-byte aligned");
    const int64_t total4 = Mp * N / 4;
    if (total4 == 0) return SCMX_OK;
    launch_pdl(res_epilogue_kernel, dim3((unsigned)((total4 + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, acc, xscale, wscale, res,
                                                                                            total4, (int)N, h);
    SCMX_LAUNCH_OK("res_epilogue_kernel");
    return SCMX_OK;
}

extern "C" int scmx_swiglu_quant(const int32_t* acc, const float* xscale, const float* wscale, int64_t Mp, int64_t F,
                                 int8_t* xq, float* xs, void* stream) {
    SCMX_REQUIRE(Mp >= 0 && F > 0 && F % 4 == 0, SCMX_EINVAL, "swiglu_quant: F=%lld must be a multiple of 4", (long long)F);
    SCMX_REQUIRE(aligned16(acc) && aligned16(wscale) && aligned16(xq), SCMX_EINVAL,
                 "swiglu_quant: buffers must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    launch_pdl(swiglu_quant_kernel, dim3((unsigned)Mp), dim3(256), 0, (cudaStream_t)stream, acc, xscale, wscale, (int)F, xq, xs);
    SCMX_LAUNCH_OK("swiglu_quant_kernel");
    return SCMX_OK;
}

extern "C" int scmx_swiglu(const uint16_t* g, const uint16_t* u, int64_t n, uint16_t* out, void* stream) {
    SCMX_REQUIRE(n >= 0, SCMX_EINVAL, "swiglu: negative length");
    if (n == 0) return SCMX_OK;
    launch_pdl(swiglu_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, g, u, n, out);
    SCMX_LAUNCH_OK("swiglu_kernel");
    return SCMX_OK;
}

extern "C" int scmx_moe_combine(const uint16_t* y, const int32_t* pos, const uint16_t* scores, const uint16_t* res,
                                const uint16_t* nw, float eps, int64_t M, int64_t Mp, int64_t K, int topk, int quant,
                                uint16_t* h, int8_t* xq, float* xs, void* stream) {
    SCMX_REQUIRE(M >= 0 && Mp >= M && K > 0 && K % 8 == 0, SCMX_EINVAL, "moe_combine: need M <= Mp and K %% 8 == 0");
    SCMX_REQUIRE(topk >= 1 && topk <= 32, SCMX_ELIMIT, "moe_combine: topk=%d outside 1..32", topk);
    SCMX_REQUIRE(aligned16(y) && aligned16(res) && aligned16(h) && (!quant || (aligned16(xq) && aligned16(nw))),
                 SCMX_EINVAL, "moe_combine: buffers must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    CombinePull pl = {};
    launch_pdl(moe_combine_kernel<32>, dim3((unsigned)Mp), dim3(256), 0, (cudaStream_t)stream, y, pos, scores, res, nw, eps, M, (int)K, topk,
               quant, h, xq, xs, pl);
    SCMX_LAUNCH_OK("moe_combine_kernel");
    return SCMX_OK;
}

extern "C" int scmx_moe_combine_pull(const void* const* y_peers, int world, int rank, int El, int64_t cap, const int32_t* esorted,
                                     const int32_t* off, const int32_t* pos, const uint16_t* scores, const uint16_t* res,
                                     const uint16_t* nw, float eps, int64_t M, int64_t Mp, int64_t K, int topk, int quant,
                                     uint16_t* h, int8_t* xq, float* xs, void* stream) {
    SCMX_REQUIRE(M >= 0 && Mp >= M && K > 0 && K % 8 == 0, SCMX_EINVAL, "moe_combine_pull: need M <= Mp and K %% 8 == 0");
    SCMX_REQUIRE(topk >= 1 && topk <= 32, SCMX_ELIMIT, "moe_combine_pull: topk=%d outside 1..32", topk);
    SCMX_REQUIRE(y_peers && world >= 1 && world <= 8 && rank >= 0 && rank < world && El >= 1 && cap >= 1 && cap < (1ll << 31) && esorted && off,
                 SCMX_EINVAL, "moe_combine_pull: bad peers / world / rank / El / cap / tables");
    SCMX_REQUIRE(aligned16(res) && aligned16(h) && (!quant || (aligned16(xq) && aligned16(nw))), SCMX_EINVAL,
                 "moe_combine_pull: buffers must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    CombinePull pl = {};
    pl.es = esorted; pl.off = off; pl.El = El; pl.cap = (int)cap; pl.rank = rank; pl.world = world;
    for (int g = 0; g < world; ++g) {
        pl.peer[g] = static_cast<const uint16_t*>(y_peers[g]);
        SCMX_REQUIRE(pl.peer[g] != nullptr && aligned16(pl.peer[g]), SCMX_EINVAL, "moe_combine_pull: buffer of rank %d is NULL or unaligned", g);
    }
    launch_pdl(moe_combine_kernel<32>, dim3((unsigned)Mp), dim3(256), 0, (cudaStream_t)stream, pl.peer[rank], pos, scores, res, nw, eps, M,
               (int)K, topk, quant, h, xq, xs, pl);
    SCMX_LAUNCH_OK("moe_combine_kernel");
    return SCMX_OK;
}

extern "C" int scmx_gather_rows(const int8_t* xq, const float* xs, const int32_t* tok, int64_t rows_q, int64_t rows_s,
                                int64_t K, int8_t* dst_q, float* dst_s, void* stream) {
    SCMX_REQUIRE(rows_q >= 0 && rows_s <= rows_q && K > 0 && K % 16 == 0, SCMX_EINVAL,
                 "gather_rows: need rows_s <= rows_q and K %% 16 == 0");
    SCMX_REQUIRE(aligned16(xq) && aligned16(dst_q), SCMX_EINVAL, "gather_rows: buffers must be 16-byte aligned");
    if (rows_q == 0) return SCMX_OK;
    launch_pdl(gather_rows_kernel, dim3((unsigned)((rows_q + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, xq, xs, tok, rows_q, rows_s, (int)K, dst_q,
               dst_s);
    SCMX_LAUNCH_OK("gather_rows_kernel");
    return SCMX_OK;
}

// Segmented-row variants: x holds nseg column segments of width K / nseg, `seg_stride` elements apart (each segment a
// row-major [M, K / nseg] matrix).  Outputs are ordinary row-major [Mp, K].
static int check_seg(const char* who, int64_t M, int64_t K, int64_t Mp, int nseg, int64_t seg_stride) {
    SCMX_REQUIRE(M >= 0 && Mp >= M && K > 0 && nseg >= 1 && K % (8 * nseg) == 0 && K <= 8192, SCMX_EINVAL,
                 "%s: need M <= Mp, K %% (8 * nseg) == 0 and K <= 8192 (M=%lld Mp=%lld K=%lld nseg=%d)", who, (long long)M,
                 (long long)Mp, (long long)K, nseg);
    SCMX_REQUIRE(seg_stride % 8 == 0 && (nseg == 1 || seg_stride >= M * (K / nseg)), SCMX_EINVAL,
                 "%s: seg_stride=%lld must be a multiple of 8 and at least M * K / nseg", who, (long long)seg_stride);
    return SCMX_OK;
}

extern "C" int scmx_act_quant_seg(const uint16_t* x, int64_t M, int64_t K, int64_t Mp, int nseg, int64_t seg_stride, int8_t* xq,
                                  float* xs, void* stream) {
    int rc = check_seg("act_quant_seg", M, K, Mp, nseg, seg_stride);
    if (rc) return rc;
    SCMX_REQUIRE(aligned16(x) && aligned16(xq), SCMX_EINVAL, "act_quant_seg: x and xq must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    launch_row_quant_warp<false>(x, nullptr, 0.0f, M, Mp, K, nseg, seg_stride, xq, xs, nullptr, (cudaStream_t)stream);
    SCMX_LAUNCH_OK("row_quant kernel");
    return SCMX_OK;
}

extern "C" int scmx_rmsnorm_quant_seg(const uint16_t* x, const uint16_t* nw, float eps, int64_t M, int64_t K, int64_t Mp,
                                      int nseg, int64_t seg_stride, int8_t* xq, float* xs, uint16_t* xn, void* stream) {
    int rc = check_seg("rmsnorm_quant_seg", M, K, Mp, nseg, seg_stride);
    if (rc) return rc;
    SCMX_REQUIRE(aligned16(x) && aligned16(nw) && aligned16(xq) && (!xn || aligned16(xn)), SCMX_EINVAL,
                 "rmsnorm_quant_seg: buffers must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    launch_row_quant_warp<true>(x, nw, eps, M, Mp, K, nseg, seg_stride, xq, xs, xn, (cudaStream_t)stream);
    SCMX_LAUNCH_OK("row_quant kernel");
    return SCMX_OK;
}


extern "C" int scmx_rot_quant(const uint16_t* x, const float* signs, int64_t M, int64_t K, int64_t Mp, int8_t* xq, float* xs,
                              void* stream) {
    SCMX_REQUIRE(M >= 0 && Mp >= M && K > 0 && K % 32 == 0 && K <= 8192, SCMX_EINVAL,
                 "rot_quant: need M <= Mp, K %% 32 == 0 and K <= 8192 (M=%lld Mp=%lld K=%lld)", (long long)M, (long long)Mp, (long long)K);
    SCMX_REQUIRE(aligned16(x) && aligned16(signs) && aligned16(xq), SCMX_EINVAL, "rot_quant: buffers must be 16-byte aligned");
    if (Mp == 0) return SCMX_OK;
    launch_pdl(rot_quant_kernel, dim3((unsigned)Mp), dim3(256), 0, (cudaStream_t)stream, x, signs, M, (int)K, xq, xs);
    SCMX_LAUNCH_OK("rot_quant_kernel");
    return SCMX_OK;
}
