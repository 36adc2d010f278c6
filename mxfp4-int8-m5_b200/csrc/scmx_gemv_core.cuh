// Instruction-level helpers of the decode GEMV kernels: streaming 128-bit loads, per-byte negation, byte permute, DP4A.
#pragma once
#include <stdint.h>

namespace scmx {

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Per-byte two's-complement negation of four INT8 without carries between bytes:
// -b = ~b + 1; the low seven bits of ~b plus one never overflow the byte, and the top bit is folded in with an XOR.
__device__ __forceinline__ uint32_t neg4(uint32_t x) {
    const uint32_t nx = ~x;
    return ((nx & 0x7F7F7F7Fu) + 0x01010101u) ^ (nx & 0x80808080u);
}

// prmt.b32 in its default mode: selector nibble bits 0-2 pick one of the eight source bytes (every selector built below
// has bit 3 of each nibble clear, so no sanitising AND is needed).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
}  // namespace scmx
