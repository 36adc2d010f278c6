// Instruction-level helpers of the decode GEMV kernels: streaming 128-bit loads, byte permute, DP4A.
#pragma once
#include <stdint.h>

namespace scmx {

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// prmt.b32 in its default mode: selector nibble bits 0-2 pick one of the eight source bytes; with bit 3 set the result byte
// is the replicated top bit of the selected byte (0x00 for values below 128), which the kernels use to zero one sign's codes.
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
