// Shared helpers of libscmx: error reporting, format upload, bf16 conversion, warp/block reductions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/scmx.h"

namespace scmx {

void set_error(const char* fmt, ...);

// ---- programmatic dependent launch ----------------------------------------------------------------------------------------
// Kernels of the chains are launched with programmatic stream serialization: a kernel may become resident while its
// predecessor drains, runs its set-up, and blocks in pdl_wait() until the predecessor has completed and flushed.  Every
// kernel performs all its reads of activations and all its writes after pdl_wait(), so by induction along the stream
// nothing earlier is still running when a kernel touches memory.
extern int g_use_pdl;
// Limit of every bounded device-side wait in nanoseconds (scmx_set_wait_limit_ns; default 2 s), handed to the kernels as an
// argument, and the per-device status word registered with scmx_set_status_word for kernels whose entry point takes none.
extern unsigned long long g_wait_limit_ns;
int32_t* device_status_word();
// Ordinal of the current device (0..63; -1 on error) and its SM count, cached per device: one process may drive several GPUs.
int current_device();
int sm_count();

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// pdl_opt: 0 = launch without the attribute whatever the process-wide switch says.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_opt(int pdl_opt, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (g_use_pdl && pdl_opt) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define SCMX_PDL_OK(name, expr)                                                              \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            ::scmx::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__));      \
            return SCMX_ECUDA;                                                                \
        }                                                                                     \
    } while (0)

#define SCMX_REQUIRE(cond, code, ...)                 \
    do {                                              \
        if (!(cond)) {                                \
            ::scmx::set_error(__VA_ARGS__);           \
            return (code);                            \
        }                                             \
    } while (0)

#define SCMX_CUDA_OK(expr)                                                                    \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            ::scmx::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));               \
            return SCMX_ECUDA;                                                                \
        }                                                                                     \
    } while (0)

#define SCMX_LAUNCH_OK(name)                                                                  \
    do {                                                                                      \
        cudaError_t e__ = cudaGetLastError();                                                 \
        if (e__ != cudaSuccess) {                                                             \
            ::scmx::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__));      \
            return SCMX_ECUDA;                                                                \
        }                                                                                     \
    } while (0)

// Device-side view of a weight format: element LUT as packed bytes, multiplier table, block geometry.
struct DevFormat {
    uint32_t mag_lo, mag_hi;     // code_mag[0..3], code_mag[4..7] as bytes
    uint32_t neg_lo, neg_hi;     // the same, negated per byte (two's complement)
    uint32_t mult4[4];           // block multipliers, 4 per word as bytes
    int block;                   // weights per block code
    int bc_bits;
    int blocks_per_byte;         // 8 / bc_bits
    int pow2;                    // 1 when mult[i] == 1 << i for every used i (the multiplier is a shift)
    int block_shift;             // log2(block) when block is a power of two, else -1 (divisions are used instead)
    int pb_shift, pb_mask;       // log2(blocks_per_byte), blocks_per_byte - 1
    int bc_shift;                // log2(bc_bits)
    uint32_t bc_mask;            // (1 << bc_bits) - 1
};

int make_dev_format(const scmx_format* fmt, DevFormat* out);

__device__ __forceinline__ float bf16_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

// float -> bfloat16 bits, round to nearest even (NaN stays NaN).
__device__ __forceinline__ uint16_t f32_to_bf16(float x) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}
__device__ __forceinline__ float rbf(float x) { return bf16_to_f32(f32_to_bf16(x)); }

// Two floats -> two bfloat16 (round to nearest even) packed in a word, `lo` in the low half.  One conversion instruction
// for two values; the conversion unit is narrow and bounded the row kernels that round several times per element
// (RMSNorm + INT8 of 2048 x 2048: 7.3 us with single conversions, 5.2 us with pairs).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t p) { return __uint_as_float(p & 0xFFFF0000u); }

// x * x as a double for a bfloat16-valued float (the product of two 8-bit significands is exact in double).
// The hardware float -> double conversion is the cheap way: rebuilding the double with integer instructions measured
// 1 us slower per RMSNorm launch of 2048 x 2048 (the integer pipe is the busier one in these kernels).
__device__ __forceinline__ double sq_f64(float f) {
    const double d = (double)f;
    return d * d;
}

// SiLU(g) * u with every step rounded to bf16: e = T(exp|g|), y = T(1/T(1+e)), sig = g<0 ? y : T(1-y),
// silu = T(g*sig), out = T(silu*u).  Same step order as e2e/sc_kernels.py:319-328.
__device__ __forceinline__ float silu_bf16(float g) {
    const float e = rbf(expf(fabsf(g)));
    const float y = rbf(__fdiv_rn(1.0f, rbf(__fadd_rn(1.0f, e))));
    const float sig = (g < 0.0f) ? y : rbf(__fsub_rn(1.0f, y));
    return rbf(__fmul_rn(g, sig));
}
__device__ __forceinline__ float swiglu_bf16(float g, float u) { return rbf(__fmul_rn(silu_bf16(g), u)); }

// y = T((float(acc) * xs) * ws), the scaling epilogue order of e2e/sc_kernels.py:101.
__device__ __forceinline__ float scale_acc(int acc, float xs, float ws) {
    return rbf(__fmul_rn(__fmul_rn((float)acc, xs), ws));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide max / sum through shared memory (blockDim.x a multiple of 32, <= 1024). `red` holds 33 entries.
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ double block_sum(double v, double* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        double t = lane < nw ? red[lane] : 0.0;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// inv = 1 / sqrt(float(sum x^2) / K + eps).  Callers accumulate the sum of squares in float64 (exact for bf16 inputs of
// ordinary dynamic range, hence independent of the reduction order); the reciprocal square root is taken in float64.
__device__ __forceinline__ float rms_inverse(double ss, int K, float eps) {
    const float m = __fadd_rn(__fdiv_rn((float)ss, (float)K), eps);
    return (float)(1.0 / sqrt((double)m));
}

// s = amax / 127, qi = s > 0 ? 1 / s : 0 in IEEE float32 (e2e/sc_kernels.py:221-222).
__device__ __forceinline__ void quant_scale(float amax, float& s, float& qi) {
    s = __fdiv_rn(amax, 127.0f);
    qi = s > 0.0f ? __fdiv_rn(1.0f, s) : 0.0f;
}
// clamp(rint(v * qi), -127, 127) with round-half-even (e2e/sc_kernels.py:225).
__device__ __forceinline__ int quant_code(float v, float qi) {
    const float r = rintf(__fmul_rn(v, qi));
    return (int)fminf(fmaxf(r, -127.0f), 127.0f);
}

// Four quantization codes packed into a word: byte j = int8(rint(v[j] * qi)).  rint is taken by adding 1.5 * 2^23, whose
// float spacing is exactly 1 (round-half-even), and the low byte of the sum's bit pattern is the two's-complement code;
// |v * qi| <= 127 by construction of qi, so no clamp is needed.  The product and the sum are rounded separately.
__device__ __forceinline__ uint32_t quant4(float v0, float v1, float v2, float v3, float qi) {
    const uint32_t b0 = __float_as_uint(__fadd_rn(__fmul_rn(v0, qi), 12582912.0f));
    const uint32_t b1 = __float_as_uint(__fadd_rn(__fmul_rn(v1, qi), 12582912.0f));
    const uint32_t b2 = __float_as_uint(__fadd_rn(__fmul_rn(v2, qi), 12582912.0f));
    const uint32_t b3 = __float_as_uint(__fadd_rn(__fmul_rn(v3, qi), 12582912.0f));
    return (b0 & 0xFFu) | ((b1 & 0xFFu) << 8) | ((b2 & 0xFFu) << 16) | (b3 << 24);
}

// Decode one 32-bit word of 8 packed codes to two words of 4 INT8 each, given per-block byte LUTs
// (positive magnitudes already multiplied by the block multiplier, and their negations).
__device__ __forceinline__ void decode_word(uint32_t w, uint32_t plo, uint32_t phi, uint32_t nlo, uint32_t nhi,
                                            uint32_t& out0, uint32_t& out1) {
    const uint32_t sel = w & 0x77777777u;
    const uint32_t ssel = ((w >> 1) & 0x44444444u) | 0x32103210u;
    const uint32_t p0 = __byte_perm(plo, phi, sel), n0 = __byte_perm(nlo, nhi, sel);
    const uint32_t p1 = __byte_perm(plo, phi, sel >> 16), n1 = __byte_perm(nlo, nhi, sel >> 16);
    out0 = __byte_perm(p0, n0, ssel);
    out1 = __byte_perm(p1, n1, ssel >> 16);
}

// Per-byte multiply of a packed magnitude LUT word by a small multiplier (every product <= 127: no carries).
__device__ __forceinline__ uint32_t lut_scale(uint32_t lut, uint32_t m) { return lut * m; }
// Per-byte two's-complement negation of bytes in 0..127.
__device__ __forceinline__ uint32_t lut_negate(uint32_t lut) {
    // -b = (b ^ 0xFF) + 1 per byte; a zero byte would carry, so bytes that are zero are left as zero.
    const uint32_t nz = ((lut | ((lut & 0x7F7F7F7Fu) + 0x7F7F7F7Fu)) & 0x80808080u) >> 7;   // 1 where byte != 0
    const uint32_t mask = nz * 0xFFu;
    return ((lut ^ mask) + nz);
}

// Block multiplier of block code bc (register-only lookup through byte permutes).
__device__ __forceinline__ uint32_t fmt_mult(const DevFormat& f, uint32_t bc) {
    const uint32_t lo = __byte_perm(f.mult4[0], f.mult4[1], bc & 7u);
    const uint32_t hi = __byte_perm(f.mult4[2], f.mult4[3], bc & 7u);
    return ((bc & 8u) ? hi : lo) & 0xFFu;
}

__device__ __forceinline__ uint32_t block_code(const uint8_t* row_bc, int blk, int bc_bits, int per_byte) {
    return (row_bc[blk / per_byte] >> (bc_bits * (blk % per_byte))) & ((1u << bc_bits) - 1u);
}
// Index of the block that holds element k of a row (shift when the block size is a power of two).
__device__ __forceinline__ int block_of(const DevFormat& f, int k) { return f.block_shift >= 0 ? (k >> f.block_shift) : (k / f.block); }
// Bit offset of block `blk` inside its byte, and the byte index: shifts only (bc_bits and codes per byte are powers of two).
__device__ __forceinline__ uint32_t block_code_fast(const DevFormat& f, const uint8_t* row_bc, int blk) {
    return (row_bc[blk >> f.pb_shift] >> ((blk & f.pb_mask) << f.bc_shift)) & f.bc_mask;
}

}  // namespace scmx
