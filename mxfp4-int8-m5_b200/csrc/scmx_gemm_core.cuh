// Device-side building blocks shared by the tcgen05 GEMM kernels of libscmx: argument block, tile scheduler, PTX wrappers
// (TMA loads, tensor-memory allocation, tcgen05.mma / commit / ld in the one-CTA and the CTA-pair forms), shared-memory and
// instruction descriptors, and the staged epilogue of one warp.
#pragma once
#include <cuda.h>
#include "scmx_common.cuh"
#include "scmx_ptx.cuh"

namespace scmx {

constexpr int BM = 128;          // rows of A per tile = TMEM lanes
constexpr int BK = 128;          // K bytes per stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;       // K per tcgen05.mma kind::i8
constexpr int EPI_WARPS = 8;
constexpr int EPI_THREADS = 32 * EPI_WARPS;
constexpr int CTA_THREADS = 64 + EPI_THREADS;   // TMA warp + MMA warp + epilogue warps

struct GemmArgs {
    int M, N, K;                 // dense: rows of xq; grouped: total sorted rows R
    int epi;
    const float* xscale;
    const float* wscale;
    const uint16_t* res;
    void* out;
    const int32_t* off;          // grouped only (E > 0)
    const int32_t* tstart;
    int E;
    int e_begin, e_end;          // grouped: experts handled by this launch; B rows are relative to e_begin
    int32_t* status;
    uint64_t wait_ns;            // limit of every mbarrier wait
    const uint16_t* silu_lut;    // 65536-entry bf16 table of silu(g) indexed by the bf16 bits of g (EPI 3)
    // EPI 1 with a return map (expert parallelism): output row r is stored at row ret_row[r] of peer_out[ret_rank[r]], the
    // buffer of the GPU the token came from, instead of row r of `out`: the GEMM's epilogue is the return exchange.
    const int32_t* ret_rank;
    int bcast;                   // > 0 (tensor parallelism): every output row is stored into peer_out[0 .. bcast) at the same row / column
    const int32_t* ret_row;
    uint16_t* peer_out[8];
};

// Barrier among the epilogue threads only (named barrier 1).
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, INT8 operands, INT32 accumulate.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base + i), registers = columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the 128-byte swizzle:
// start address >> 4 in bits [0,14); leading byte offset (unused for swizzled K-major) = 1 in [16,30);
// stride byte offset = 1024 (eight rows) >> 4 in [32,46); descriptor version 1 in [46,48); layout 2 = SWIZZLE_128B
// in [61,64).  Advancing K by 32 bytes inside the swizzle row adds 2 to the start-address field.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::i8: D = S32 (2 at [4,6)), A and B signed INT8 (1 at [7,10) and [10,13)), both K-major
// (bits 15, 16 zero), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- tile scheduler ---------------------------------------------------------------------------------------------------
struct Tile {
    int row0;        // first A row (TMA coordinate; also first output row)
    int row_end;     // rows >= row_end are not stored
    int n0;          // first output column
    int brow;        // first B row (TMA coordinate)
    int wrow;        // index of wscale[n0]
};

template <int BN>
__device__ __forceinline__ int num_tiles(const GemmArgs& a, int& tiles_m, int& slot0) {
    const int tiles_n = (a.N + BN - 1) / BN;
    if (a.E == 0) {
        tiles_m = (a.M + BM - 1) / BM;
        slot0 = 0;
    } else {
        slot0 = a.tstart[a.e_begin];
        tiles_m = a.tstart[a.e_end] - slot0;
    }
    return tiles_m * tiles_n;
}

template <int BN>
__device__ __forceinline__ Tile get_tile(const GemmArgs& a, int t, int tiles_m, int slot0) {
    Tile tl;
    // Tiles are visited in bands of `gm` M tiles: inside a band m runs fastest, then n, then the next band.  The CTAs that run
    // at the same time then share a few B tiles (one per expert and column) and the A rows of a band stay in L2 until all
    // columns have used them; with plain m-fastest order over thousands of sorted rows every column sweep re-read A from
    // DRAM (grouped gate|up GEMM: 689 MB read for 335 MB of operands).  Two waves of CTAs per band.
    const int tiles_n = (a.N + BN - 1) / BN;
    // (dense launches have at most a few dozen M tiles and L2-resident operands: one band)
    const int gm_full = a.E == 0 ? tiles_m : max(1, (2 * (int)gridDim.x + tiles_n - 1) / tiles_n);
    const int band = t / (gm_full * tiles_n), r = t - band * gm_full * tiles_n;
    const int gm = min(gm_full, tiles_m - band * gm_full);
    const int nt = r / gm, mt = band * gm_full + r - nt * gm;
    tl.n0 = nt * BN;
    if (a.E == 0) {
        tl.row0 = mt * BM;
        tl.row_end = a.M;
        tl.brow = tl.n0;
        tl.wrow = tl.n0;
    } else {
        const int s = slot0 + mt;
        int lo = a.e_begin, hi = a.e_end;      // largest e in [e_begin, e_end) with tstart[e] <= s
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (a.tstart[mid] <= s) lo = mid; else hi = mid;
        }
        tl.row0 = a.off[lo] + (s - a.tstart[lo]) * BM;
        tl.row_end = a.off[lo + 1];
        tl.brow = (lo - a.e_begin) * a.N + tl.n0;
        tl.wrow = lo * a.N + tl.n0;
    }
    return tl;
}

// ---- epilogue of 32 consecutive columns of one row ----------------------------------------------------------------------
__device__ __forceinline__ float scale2(uint32_t acc, float xs, float w) { return __fmul_rn(__fmul_rn((float)(int)acc, xs), w); }

// ---- epilogue of one warp: 32 rows x BN/2 accumulator columns ----------------------------------------------------------------
// tcgen05.ld hands every thread ONE row (32 consecutive columns per load), so storing straight from registers would write 32
// different rows per instruction, 16 bytes each.  Instead the converted values go through a small shared-memory staging area
// (per warp 32 rows x 128 bytes, pitch 144 so that both the row-per-thread writes and the row-wise reads are free of bank
// conflicts) and leave as full 128-byte lines: 4 rows per store instruction.  The residual of EPI 2 comes in the same way
// (coalesced loads issued before the accumulators are awaited, staged, read back row-per-thread).
//   EPI 0: INT32; EPI 1: T((float(acc)*xs)*ws); EPI 2: T(res + T(...)); EPI 3: per 4 columns [g0,g1,u0,u1] ->
//   T(silu(T(g)) * T(u)) x 2 with silu(g) = T(g * sigmoid_T(g)) read from a 65536-entry table indexed by the bf16 bits of g
//   (built once per device by evaluating the step-by-step bf16 formula for every gate value).
constexpr int EPI_PITCH = 144;
constexpr int EPI_STAGE_WARP = 32 * EPI_PITCH;          // 4608 bytes per epilogue warp
constexpr int EPI_STAGE_BYTES = EPI_WARPS * EPI_STAGE_WARP;

// Start of output row `row` (row_bytes per row): the local output, or with a return map the buffer of the GPU the row's token
// came from; null when the map is inconsistent (nothing is stored then).
__device__ __forceinline__ uint8_t* out_row_ptr(const GemmArgs& a, int row, size_t row_bytes) {
    if (a.ret_rank != nullptr) {
        const int rr = a.ret_rank[row], r2 = a.ret_row[row];
        if (rr < 0 || rr >= 8 || r2 < 0) return nullptr;
        uint16_t* base = a.peer_out[rr];
        return base == nullptr ? nullptr : reinterpret_cast<uint8_t*>(base) + (size_t)r2 * row_bytes;
    }
    return reinterpret_cast<uint8_t*>(a.out) + (size_t)row * row_bytes;
}

// Staged 32 x 128 bytes -> global memory; `valid` = bytes of the unit that lie inside the matrix (a multiple of 16).
template <bool BCAST = false>
__device__ __forceinline__ void epi_drain(const GemmArgs& a, const uint8_t* stg, int lane, int row0, int row_end, size_t row_bytes,
                                          size_t col_byte0, int valid) {
    const int piece = lane & 7, rsub = lane >> 3;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int rl = 4 * i + rsub;
        const uint4 v = *reinterpret_cast<const uint4*>(stg + rl * EPI_PITCH + piece * 16);
        const int row = row0 + rl;
        if (row < row_end && piece * 16 < valid) {
            if (BCAST) {
                // the all-gather of tensor parallelism issued from the epilogue: the same full line into every GPU's buffer
                const size_t o = (size_t)row * row_bytes + col_byte0 + piece * 16;
#pragma unroll
                for (int g = 0; g < 8; ++g)
                    if (g < a.bcast) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.peer_out[g]) + o) = v;
            } else {
                uint8_t* p = out_row_ptr(a, row, row_bytes);
                if (p != nullptr) *reinterpret_cast<uint4*>(p + col_byte0 + piece * 16) = v;
            }
        }
    }
}

// Coalesced load of the residual of one 64-column unit (32 rows x 128 bytes) into registers, in the staging layout.
__device__ __forceinline__ void epi_load_res(const GemmArgs& a, uint4 (&rp)[8], int lane, int row0, int row_end, int n_unit) {
    const int piece = lane & 7, rsub = lane >> 3;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = row0 + 4 * i + rsub, col = n_unit + piece * 8;
        rp[i] = make_uint4(0, 0, 0, 0);
        if (row < row_end && col < a.N) rp[i] = __ldg(reinterpret_cast<const uint4*>(a.res + (size_t)row * a.N + col));
    }
}
__device__ __forceinline__ void epi_stage_res(uint8_t* stg, const uint4 (&rp)[8], int lane) {
    const int piece = lane & 7, rsub = lane >> 3;
#pragma unroll
    for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(stg + (4 * i + rsub) * EPI_PITCH + piece * 16) = rp[i];
}

// One 32-column chunk of the thread's row -> staged output bytes.  ws: the chunk's 32 staged weight scales.
__device__ __forceinline__ void epi_convert(const GemmArgs& a, const uint32_t (&r)[32], const float* ws, float xs, uint8_t* my, int c) {
    if (a.epi == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) reinterpret_cast<uint4*>(my)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    } else if (a.epi == 3) {
        uint32_t pk[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 w4 = *reinterpret_cast<const float4*>(ws + 4 * g);
            const uint32_t gg = pack_bf16x2(scale2(r[4 * g], xs, w4.x), scale2(r[4 * g + 1], xs, w4.y));
            const uint32_t uu = pack_bf16x2(scale2(r[4 * g + 2], xs, w4.z), scale2(r[4 * g + 3], xs, w4.w));
            const float s0 = __uint_as_float((uint32_t)__ldg(a.silu_lut + (gg & 0xFFFFu)) << 16);
            const float s1 = __uint_as_float((uint32_t)__ldg(a.silu_lut + (gg >> 16)) << 16);
            pk[g] = pack_bf16x2(__fmul_rn(s0, bf16_lo(uu)), __fmul_rn(s1, bf16_hi(uu)));
        }
        uint4* o = reinterpret_cast<uint4*>(my + 32 * c);                 // 16 outputs = 32 bytes per chunk
        o[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        o[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    } else {
        uint4* o = reinterpret_cast<uint4*>(my + 64 * (c & 1));           // 32 outputs = 64 bytes per chunk, two chunks per unit
        uint32_t pk[16];
        if (a.epi == 2) {
            uint32_t rr[16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = o[j];                                      // the staged residual of this row
                rr[4 * j] = v.x; rr[4 * j + 1] = v.y; rr[4 * j + 2] = v.z; rr[4 * j + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float2 w2 = *reinterpret_cast<const float2*>(ws + 2 * j);
                const uint32_t y = pack_bf16x2(scale2(r[2 * j], xs, w2.x), scale2(r[2 * j + 1], xs, w2.y));
                pk[j] = pack_bf16x2(__fadd_rn(bf16_lo(rr[j]), bf16_lo(y)), __fadd_rn(bf16_hi(rr[j]), bf16_hi(y)));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float2 w2 = *reinterpret_cast<const float2*>(ws + 2 * j);
                pk[j] = pack_bf16x2(scale2(r[2 * j], xs, w2.x), scale2(r[2 * j + 1], xs, w2.y));
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    }
}

// The warp's part of a tile.  taddr: TMEM address of its lane quarter and column half; ws: staged scales of that half;
// row0 / row_end: its 32 rows and the first row not to store; n0: first accumulator column of its half; rp: the residual of
// the first 64-column unit, loaded by the caller (epi_load_res) before it waited for the accumulators.
// PIPE: keep the next chunk's tensor-memory load in flight while a chunk is converted (64 registers of accumulators instead
// of 32); kernels with many other warps per CTA run it without.
template <int BN, bool PIPE = true, bool BCAST = false>
__device__ __forceinline__ void epilogue_warp(const GemmArgs& a, uint32_t taddr, const float* ws, int row0, int row_end, int n0,
                                              uint8_t* stg, int lane, float xs, uint4 (&rp)[8]) {
    constexpr int CHUNKS = BN / 64;           // 32-column chunks per warp
    uint8_t* my = stg + lane * EPI_PITCH;
    uint32_t r0[32], r1[PIPE ? 32 : 1];
    tmem_ld32(taddr, r0);
    if (a.epi == 2) {
        epi_stage_res(stg, rp, lane);
        __syncwarp();
        if (CHUNKS > 2) epi_load_res(a, rp, lane, row0, row_end, n0 + 64);
    }
    tmem_ld_wait();
#pragma unroll
    for (int c = 0; c < CHUNKS; c += 2) {
        if (PIPE) tmem_ld32(taddr + (c + 1) * 32, reinterpret_cast<uint32_t(&)[32]>(r1));
        epi_convert(a, r0, ws + c * 32, xs, my, c);
        if (a.epi == 0) {
            __syncwarp();
            epi_drain<BCAST>(a, stg, lane, row0, row_end, (size_t)a.N * 4, (size_t)(n0 + c * 32) * 4, min(128, (a.N - (n0 + c * 32)) * 4));
            __syncwarp();
        }
        if (!PIPE) tmem_ld32(taddr + (c + 1) * 32, r0);
        tmem_ld_wait();
        if (PIPE && c + 2 < CHUNKS) tmem_ld32(taddr + (c + 2) * 32, r0);
        epi_convert(a, PIPE ? reinterpret_cast<uint32_t(&)[32]>(r1) : r0, ws + (c + 1) * 32, xs, my, c + 1);
        if (a.epi == 0) {
            __syncwarp();
            epi_drain<BCAST>(a, stg, lane, row0, row_end, (size_t)a.N * 4, (size_t)(n0 + (c + 1) * 32) * 4, min(128, (a.N - (n0 + (c + 1) * 32)) * 4));
            __syncwarp();
        } else if (a.epi != 3) {
            __syncwarp();
            epi_drain<BCAST>(a, stg, lane, row0, row_end, (size_t)a.N * 2, (size_t)(n0 + c * 32) * 2, min(128, (a.N - (n0 + c * 32)) * 2));
            __syncwarp();
            if (a.epi == 2 && c + 2 < CHUNKS) {
                epi_stage_res(stg, rp, lane);
                __syncwarp();
            }
        }
        if (!PIPE && c + 2 < CHUNKS) tmem_ld32(taddr + (c + 2) * 32, r0);
        if (c + 2 < CHUNKS) tmem_ld_wait();
    }
    if (a.epi == 3) {
        __syncwarp();
        epi_drain<BCAST>(a, stg, lane, row0, row_end, (size_t)a.N, (size_t)n0, min(32 * CHUNKS, a.N - n0));
        __syncwarp();
    }
}

// ---- CTA-pair (cta_group::2) forms -------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: the data lands in this CTA's shared memory, the bytes are counted on an mbarrier that may
// live in the other CTA of the pair (`bar` is a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the mbarrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

// ---- host-side helpers defined in scmx_gemm.cu -------------------------------------------------------------------------------
int silu_lut_ptr(cudaStream_t st, const uint16_t** out);
int make_map_u8(CUtensorMap* map, const void* ptr, int64_t rows, int64_t row_bytes, int box_bytes, int box_rows, int swizzle_bytes);
int check_common(const char* who, int64_t N, int64_t K, int epi, const float* xscale, const float* wscale, const void* out,
                 const int32_t* status);

}  // namespace scmx
