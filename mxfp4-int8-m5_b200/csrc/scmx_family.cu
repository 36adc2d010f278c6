// Quantizer of the integer-exact 4-bit format family  w[n,k] = base[n] * mult[n, k/block] * (+-code_mag[idx])
// in float32 arithmetic, bit-compatible with the reference's NumPy implementation (sim/formats.py:57-107) followed by
// its packer (e2e/pack_format.py:53-76).
//
// One CTA per row, one thread per block.  For each of `base_grid` candidate row bases
// (base_hi * float32(2^(-j/base_grid)), base_hi = rowmax / (max mult * max code)), every block picks the multiplier
// with the smallest squared error (first minimum), the row total decides strictly-better bases.  All sums follow
// NumPy's pairwise order for contiguous float32 axes of length 8..128 (eight strided partial sums, fixed tree) and
// every product / quotient is rounded separately (no fused multiply-add).
#include <math.h>
#include "scmx_common.cuh"

namespace scmx {

struct FamilyArgs {
    float cb[8];        // code magnitudes
    float mids[7];      // midpoints between consecutive magnitudes
    float mu[16];       // multipliers
    float grid[16];     // float32(2^(-j / base_grid))
    int n_mult, base_grid, block, bc_bits, per_byte;
};

__device__ __forceinline__ int cb_index(const FamilyArgs& a, float v) {
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 7; ++i) idx += (a.mids[i] < v);
    return idx;
}
// sign(x) * cb[searchsorted(mids, min(|x|, cmax))]
__device__ __forceinline__ float cb_round(const FamilyArgs& a, float x, int* idx_out = nullptr) {
    const float m = fminf(fabsf(x), a.cb[7]);
    const int idx = cb_index(a, m);
    if (idx_out) *idx_out = idx;
    const float c = a.cb[idx];
    return x > 0.0f ? c : (x < 0.0f ? -c : 0.0f * c);
}

__device__ __forceinline__ float tree8(const float (&r)[8]) {
    return __fadd_rn(__fadd_rn(__fadd_rn(r[0], r[1]), __fadd_rn(r[2], r[3])),
                     __fadd_rn(__fadd_rn(r[4], r[5]), __fadd_rn(r[6], r[7])));
}

__device__ __forceinline__ float block_err(const FamilyArgs& a, const float* wb, float s) {
    float r[8];
    for (int c = 0; c < a.block; c += 8) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const float w = wb[c + t];
            const float d = __fsub_rn(__fmul_rn(cb_round(a, __fdiv_rn(w, s)), s), w);
            const float sq = __fmul_rn(d, d);
            r[t] = c == 0 ? sq : __fadd_rn(r[t], sq);
        }
    }
    return tree8(r);
}

__global__ void __launch_bounds__(128) family_kernel(const float* __restrict__ w, int K, const FamilyArgs a,
                                                     uint32_t* __restrict__ codes, uint8_t* __restrict__ bcodes,
                                                     float* __restrict__ wscale, int8_t* __restrict__ qw) {
    extern __shared__ float s_w[];            // the row, then per-block picked errors, then per-block multiplier ids
    __shared__ float red[33];
    __shared__ float s_base, s_best;
    __shared__ int s_better;
    const int nb = K / a.block;
    float* s_err = s_w + K;
    int* s_m = reinterpret_cast<int*>(s_err + nb);
    const int64_t n = blockIdx.x;
    const int b = threadIdx.x;
    float amax = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = w[n * K + k];
        s_w[k] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    amax = block_max(amax, red);     // also orders the s_w writes
    if (amax == 0.0f) amax = 1.0f;
    const float base_hi = __fdiv_rn(amax, __fmul_rn(a.mu[a.n_mult - 1], a.cb[7]));
    if (threadIdx.x == 0) { s_best = INFINITY; s_base = base_hi; }
    int best_m = 0;
    __syncthreads();
    for (int j = 0; j < a.base_grid; ++j) {
        const float base = __fmul_rn(base_hi, a.grid[j]);
        int mi = 0;
        if (b < nb) {
            float e_best = 0.0f;
            for (int i = 0; i < a.n_mult; ++i) {
                const float e = block_err(a, s_w + b * a.block, __fmul_rn(base, a.mu[i]));
                if (i == 0 || e < e_best) { e_best = e; mi = i; }
            }
            s_err[b] = e_best;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float r[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) r[t] = s_err[t];
            for (int i = 8; i < nb; i += 8) {
#pragma unroll
                for (int t = 0; t < 8; ++t) r[t] = __fadd_rn(r[t], s_err[i + t]);
            }
            const float tot = tree8(r);
            s_better = tot < s_best;
            if (s_better) { s_best = tot; s_base = base; }
        }
        __syncthreads();
        if (s_better) best_m = mi;
        __syncthreads();
    }
    const float base = s_base;
    if (threadIdx.x == 0) wscale[n] = base;
    if (b < nb) s_m[b] = best_m;
    __syncthreads();
    if (b >= nb) return;
    const float m = a.mu[best_m];
    const float s = __fmul_rn(base, m);
    const float* wb = s_w + b * a.block;
    for (int c = 0; c < a.block; c += 8) {
        uint32_t word = 0, q0 = 0, q1 = 0;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            int idx;
            const float cv = cb_round(a, __fdiv_rn(wb[c + t], s), &idx);
            const float qf = __fmul_rn(cv, m);
            const int qi = (int)qf;
            word |= (uint32_t)(idx | ((qf < 0.0f) ? 8 : 0)) << (4 * t);
            if (t < 4) q0 |= ((uint32_t)qi & 0xFFu) << (8 * t);
            else q1 |= ((uint32_t)qi & 0xFFu) << (8 * (t - 4));
        }
        const int64_t wi = (n * K + (int64_t)b * a.block + c) / 8;
        codes[wi] = word;
        if (qw) reinterpret_cast<uint2*>(qw)[wi] = make_uint2(q0, q1);
    }
    if (b % a.per_byte == 0) {
        uint32_t byte = 0;
        for (int i = 0; i < a.per_byte; ++i) byte |= (uint32_t)s_m[b + i] << (a.bc_bits * i);
        bcodes[n * (nb / a.per_byte) + b / a.per_byte] = (uint8_t)byte;
    }
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_quantize_family(const float* w, int64_t N, int64_t K, const scmx_format* fmt, int base_grid,
                                    uint32_t* codes, uint8_t* bcodes, float* wscale, int8_t* qw, void* stream) {
    DevFormat f;
    int rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    SCMX_REQUIRE(base_grid >= 1 && base_grid <= 16, SCMX_ELIMIT, "quantize_family: base_grid=%d outside 1..16", base_grid);
    SCMX_REQUIRE(N >= 0 && K > 0 && K % fmt->block == 0, SCMX_EINVAL, "quantize_family: K=%lld not a multiple of block=%d",
                 (long long)K, fmt->block);
    const int nb = (int)(K / fmt->block);
    SCMX_REQUIRE(nb % 8 == 0 && nb >= 8 && nb <= 128 && nb % f.blocks_per_byte == 0, SCMX_ELIMIT,
                 "quantize_family: %d blocks per row; need a multiple of 8 in 8..128", nb);
    FamilyArgs a = {};
    for (int i = 0; i < 8; ++i) a.cb[i] = (float)fmt->code_mag[i];
    for (int i = 0; i < 7; ++i) {
        SCMX_REQUIRE(fmt->code_mag[i + 1] > fmt->code_mag[i], SCMX_EFORMAT, "quantize_family: code_mag must be ascending");
        a.mids[i] = (a.cb[i + 1] + a.cb[i]) / 2.0f;
    }
    for (int i = 0; i < fmt->n_mult; ++i) {
        SCMX_REQUIRE(i == 0 || fmt->mult[i] > fmt->mult[i - 1], SCMX_EFORMAT, "quantize_family: mult must be ascending");
        a.mu[i] = (float)fmt->mult[i];
    }
    for (int j = 0; j < base_grid; ++j) a.grid[j] = (float)pow(2.0, -(double)j / (double)base_grid);
    a.n_mult = fmt->n_mult; a.base_grid = base_grid; a.block = fmt->block; a.bc_bits = fmt->bc_bits;
    a.per_byte = f.blocks_per_byte;
    if (N == 0) return SCMX_OK;
    const size_t smem = (size_t)K * 4 + (size_t)nb * 8;
    SCMX_REQUIRE(smem <= 48 * 1024, SCMX_ELIMIT, "quantize_family: K=%lld too large", (long long)K);
    family_kernel<<<(unsigned)N, 128, smem, (cudaStream_t)stream>>>(w, (int)K, a, codes, bcodes, wscale, qw);
    SCMX_LAUNCH_OK("family_kernel");
    return SCMX_OK;
}
