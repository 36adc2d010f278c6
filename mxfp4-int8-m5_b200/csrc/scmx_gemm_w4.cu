// W4A8 GEMM straight from the packed 4-bit codes: the weight tile is expanded to INT8 inside the K loop, in shared memory,
// so the decoded weights never exist in global memory (the structure of the reference's grouped kernel,
// e2e/sc_moe.py:47-69, and of its single-pass dense kernel, kernels/w4a8.metal:78-155).  Dense and grouped (per-expert row
// segments) problems; tcgen05.mma kind::i8 on CTA pairs as in gemm_i8_pair_kernel.
//
// A pair of CTAs shares a 256 x 256 output tile; per 128-wide K block each CTA needs ITS 128 rows of A (16 KB INT8 by TMA)
// and ITS 128 of the tile's 256 weight rows, which arrive as 8 KB of packed codes (TMA, 64-byte swizzle so that a thread can
// read "its" weight row without bank conflicts) and are expanded by eight unpack warps, two threads per weight row:
//     packed row (64 B) -> 16 code words -> byte-permute lookups of the magnitudes of positive and of negative codes
//     (the sign bit of a code switches the permute to "replicate the top bit of the selected byte", i.e. to zero) ->
//     signed bytes = ((P | 0x80..) - Q) ^ 0x80.. -> 128 B of INT8 written into the 128-byte-swizzled operand stage
// with the block multiplier folded into the lookup table per block.  Because the pair splits the weight rows, each SM
// expands half a tile per K block - about the time its tensor core needs for the MMAs of that block - and both run
// concurrently.  Roles per CTA (576 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only), warps 2..9 epilogue,
// warps 10..17 unpack (thread = one weight row x half a K block).  Barriers per stage: loaded (TMA bytes of this CTA landed;
// awaited by its unpack warps), full (lives in the leader: its 8 unpack warps arrive after their stores and a proxy fence,
// the peer's 8 warps each send a 16-byte asynchronous copy that completes on it; awaited by the MMA thread), empty (both
// CTAs, signalled by the leader's tcgen05.commit).  All waits are bounded.
// Where a row segment spans more than one row tile the kernel works on "super tiles" (MT = 2): 512 rows x 128 columns, the two
// row tiles sharing every expanded weight tile (half the expansion per MMA; the thread layout becomes weight row x quarter of
// a K block and a stage holds two activation tiles).
// Measured on B200 (gate|up 2048 x 12288 x 2048): 1600 cycles per K block with 256 x 256 tiles, 1277 with super tiles, against
// 512 cycles of MMA and ~660 of the INT8 kernel; halving the expansion work removed only a fifth, and neither a second block in
// flight per unpack warp group nor separate rings for activations / packed codes / expanded tiles shortened it (both
// measured: equal and slower).  The kernel wins where an expert sees few rows (the decoded weights would be used once) and
// loses to decode-then-GEMM where every decoded tile is reused by many row tiles, which is the reference's own rule for
// choosing between its two forms (e2e/fused_olmoe.py:205).
#include "scmx_gemm_core.cuh"
#include "scmx_gemv_core.cuh"

namespace scmx {

constexpr int W4_STAGES = 4;
constexpr int W4_BN = 256;
constexpr int W4_UNPACK_WARPS = 8;
constexpr int W4_THREADS = CTA_THREADS + 32 * W4_UNPACK_WARPS;      // 576
constexpr int W4_MAX_E = 512;                                       // pair-tile table in shared memory

// MT = row tiles (of 256 rows per CTA pair) that share one expanded weight tile.  MT = 1: 256 x 256 output tiles.  MT = 2:
// "super tiles" of 512 rows x 128 columns: every expanded K block of 128 weight rows feeds the MMAs of two row tiles, so the
// expansion per MMA halves; the two accumulators of a super tile sit side by side in tensor memory (2 x 128 columns) and the
// second row tile is skipped where a segment ends inside the first.
template <int MT>
struct W4SmemT {
    static constexpr int BN = W4_BN / MT;                   // output columns of a tile
    static constexpr int BH = BN / 2;                       // weight rows expanded by one CTA
    static constexpr int A_TILE = BM * BK;                  // 16 KB per row tile
    static constexpr int A_BYTES = MT * A_TILE;
    static constexpr int B_BYTES = BH * BK;                 // INT8, written by the unpack warps
    static constexpr int P_BYTES = BH * (BK / 2);           // packed codes
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + P_BYTES;
    static constexpr int BAR_OFF = W4_STAGES * STAGE_BYTES;                 // loaded[S], full[S], empty[S], tfull[2], tempty[2]
    static constexpr int MISC_OFF = BAR_OFF + 8 * (3 * W4_STAGES + 4);
    static constexpr int WS_OFF = MISC_OFF + 16;
    static constexpr int EPI_OFF = WS_OFF + 2 * W4_BN * 4;
    static constexpr int PT_OFF = EPI_OFF + EPI_STAGE_BYTES;               // tile starts per expert [W4_MAX_E + 1]
    static constexpr int SIG_OFF = PT_OFF + 4 * (W4_MAX_E + 4);             // 16-byte aligned: 8 x 16 B signal source, 8 x 16 B sink
    static constexpr int TOTAL = SIG_OFF + 256 + 1024;
};
static_assert(W4SmemT<1>::TOTAL <= 232448 && W4SmemT<2>::TOTAL <= 232448, "shared memory of the packed-weight GEMM exceeds 227 KB");
static_assert(W4SmemT<1>::STAGE_BYTES % 1024 == 0 && W4SmemT<2>::STAGE_BYTES % 1024 == 0, "stages must keep the swizzle alignment");

struct W4Args {
    GemmArgs g;                   // M / R, N, K, epilogue, scales, output, expert segments (off; tstart unused), status
    const uint8_t* bcodes;        // [rows, bc_row] block codes
    int bc_row;                   // block-code bytes per weight row
    int field_bits;               // block-code bits per 128-wide K block: 8, 16 or 32
    DevFormat f;
};

struct W4Tile {
    int nm;          // row tiles of this (super) tile that hold rows: 1 .. MT
    int row0;        // first A row of this CTA (row tile 0; row tile m starts 256 m rows further)
    int row_end;     // rows >= row_end are not stored
    int n0;          // first output column of the tile
    int wbase;       // index of the tile's first weight row (expert * N + n0): wscale, packed rows and block codes
};

// Signed INT8 of the 8 codes of word w: o0 = codes 0..3, o1 = codes 4..7; (mlo, mhi) = magnitudes x block multiplier.
__device__ __forceinline__ void decode_word_pq(uint32_t w, uint32_t mlo, uint32_t mhi, uint32_t& o0, uint32_t& o1) {
    const uint32_t wx = w ^ 0x88888888u, H = 0x80808080u;
    const uint32_t p0 = prmt(mlo, mhi, w), q0 = prmt(mlo, mhi, wx);
    const uint32_t p1 = prmt(mlo, mhi, w >> 16), q1 = prmt(mlo, mhi, wx >> 16);
    o0 = ((p0 | H) - q0) ^ H;       // per byte p - q: at most one of them is non-zero, the bias keeps borrows inside the byte
    o1 = ((p1 | H) - q1) ^ H;
}

template <bool POW2, int MT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(W4_THREADS, 1)
    gemm_w4_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmP, const W4Args wa) {
    using L = W4SmemT<MT>;
    constexpr int STAGES = W4_STAGES, BN = L::BN, BH = L::BH;
    constexpr int SUPER = MT * 2 * BM;                      // rows of a (super) tile
    const GemmArgs& a = wa.g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_loaded = sbase + L::BAR_OFF, bar_full = bar_loaded + 8 * STAGES, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC_OFF + 4);
    float* ws_stage = reinterpret_cast<float*>(smem + L::WS_OFF);
    int* ptile = reinterpret_cast<int*>(smem + L::PT_OFF);            // grouped: pair-tile start of every expert
    constexpr uint32_t ACC_COLS = MT * BN;                  // 256 either way: two accumulator sets fill tensor memory
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_loaded + 8 * s, 1);
            mbar_init(bar_full + 8 * s, W4_UNPACK_WARPS);          // the leader's unpack warps; the peer's count as bytes
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 2 * EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish2();
    }
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();        // expert offsets, activations and scales come from earlier kernels of the stream

    // ---- tile table.  Dense: tiles_m = ceil(M / 256).  Grouped: expert e owns ceil(rows_e / 256) pair tiles.
    const int tiles_n = (a.N + BN - 1) / BN;
    int tiles_m;
    if (a.E == 0) {
        tiles_m = (a.M + SUPER - 1) / SUPER;
    } else {
        if (warp == 2) {
            int run = 0;
            for (int b0 = 0; b0 < a.E; b0 += 32) {
                const int e = b0 + lane;
                const int c = e < a.E ? (a.off[e + 1] - a.off[e] + SUPER - 1) / SUPER : 0;
                int sc = c;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, sc, d);
                    if (lane >= d) sc += v;
                }
                if (e < a.E) ptile[e] = run + sc - c;
                run += __shfl_sync(0xffffffffu, sc, 31);
            }
            if (lane == 0) ptile[a.E] = run;
        }
        __syncthreads();
        tiles_m = ptile[a.E];
    }
    const int total = tiles_m * tiles_n;
    const int num_kb = (a.K + BK - 1) / BK;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    // tiles are visited in bands of gm pair-rows, m fastest inside a band, then n: the CTAs running together share a few
    // weight tiles through L2 and the A rows of a band stay there until every column has used them
    const int gm_full = a.E == 0 ? tiles_m : max(1, (2 * npairs + tiles_n - 1) / tiles_n);
    auto get_tile = [&](int t) {
        W4Tile tl;
        const int band = t / (gm_full * tiles_n), r = t - band * gm_full * tiles_n;
        const int gm = min(gm_full, tiles_m - band * gm_full);
        const int nt = r / gm, mt = band * gm_full + r - nt * gm;
        tl.n0 = nt * BN;
        int base;                                 // first row of the (super) tile
        if (a.E == 0) {
            base = mt * SUPER;
            tl.row_end = a.M;
            tl.wbase = tl.n0;
        } else {
            int lo = 0, hi = a.E;                 // largest e with ptile[e] <= mt
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (ptile[mid] <= mt) lo = mid; else hi = mid;
            }
            base = a.off[lo] + (mt - ptile[lo]) * SUPER;
            tl.row_end = a.off[lo + 1];
            tl.wbase = lo * a.N + tl.n0;
        }
        tl.row0 = base + (int)rank * BM;
        tl.nm = (MT == 2 && base + 2 * BM < tl.row_end) ? 2 : 1;
        return tl;
    };
    const uint32_t full_leader = mapa_u32(bar_full, 0), tempty_leader = mapa_u32(bar_tempty, 0);
    int fail = 0;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: this CTA's A rows and packed weight rows
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = pair; t < total && fail == 0; t += npairs) {
                const W4Tile tl = get_tile(t);
                const int prow = tl.wbase + (int)rank * BH;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (int w = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, a.wait_ns)) { fail = w == 1 ? 1 : -1; break; }
                    const uint32_t sa = sbase + stage * L::STAGE_BYTES, sp = sa + L::A_BYTES + L::B_BYTES;
                    mbar_expect_tx(bar_loaded + 8 * stage, tl.nm * L::A_TILE + L::P_BYTES);
                    tma_load_2d(sa, &tmA, kb * BK, tl.row0, bar_loaded + 8 * stage);
                    if (MT == 2 && tl.nm == 2) tma_load_2d(sa + L::A_TILE, &tmA, kb * BK, tl.row0 + 2 * BM, bar_loaded + 8 * stage);
                    tma_load_2d(sp, &tmP, kb * (BK / 2), prow, bar_loaded + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc(2 * BM, BN);
            int stage = 0;
            uint32_t phase = 0, acc = 0, acc_phase = 0;
            for (int t = pair; t < total && fail == 0; t += npairs) {
                const int nm = MT == 2 ? get_tile(t).nm : 1;
                if (int w = mbar_wait_cluster(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, a.wait_ns)) { fail = w == 1 ? 2 : -1; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (int w = mbar_wait_cluster(bar_full + 8 * stage, phase, abort_flag, a.wait_ns)) { fail = w == 1 ? 3 : -1; break; }
                    tc_fence_after();
                    const uint32_t sa = sbase + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
                    const uint64_t db = umma_desc(sb);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        if (m < nm) {                       // the row tiles of a super tile share the expanded weight tile
                            const uint64_t da = umma_desc(sa + m * L::A_TILE);
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k)
                                umma_i8_pair(d_tmem + m * BN, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc,
                                             (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit_pair(bar_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (fail) break;
                umma_commit_pair(bar_tfull + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else if (warp < 2 + EPI_WARPS) {
        // ------------------------------------------------ epilogue warps
        const int q = warp & 3;
        const int chalf = (warp - 2) >> 2;
        const int et = threadIdx.x - 64;
        uint32_t acc = 0, acc_phase = 0;
        for (int t = pair; t < total && fail == 0; t += npairs) {
            const W4Tile tl = get_tile(t);
            float* ws = ws_stage + acc * W4_BN;
            if (a.epi != 0) {
                for (int i = et; i < BN; i += EPI_THREADS) ws[i] = (tl.n0 + i < a.N) ? a.wscale[tl.wbase + i] : 0.0f;
            }
            // a warp converts 128 accumulator columns of 32 rows: MT = 1: column half `chalf` of the tile's rows; MT = 2: all 128
            // columns of row tile `chalf`.  Either way they are columns chalf * 128 .. + 127 of the accumulator set.
            const int mtile = MT == 2 ? chalf : 0, coff = MT == 2 ? 0 : chalf * 128;
            const int wrow0 = tl.row0 + mtile * 2 * BM + 32 * q;
            const float xs = (a.epi != 0 && wrow0 + lane < tl.row_end) ? a.xscale[wrow0 + lane] : 0.0f;
            uint4 rp[8];
            if (a.epi == 2 && mtile < tl.nm) epi_load_res(a, rp, lane, wrow0, tl.row_end, tl.n0 + coff);
            if (int w = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, a.wait_ns)) fail = w == 1 ? 4 : -1;
            epilogue_bar();
            if (*abort_flag) { if (!fail) fail = -1; break; }
            tc_fence_after();
            if (mtile < tl.nm)
                epilogue_warp<256, false>(a, tmem_base + acc * ACC_COLS + chalf * 128 + ((uint32_t)(32 * q) << 16), ws + coff, wrow0,
                                          tl.row_end, tl.n0 + coff, smem + L::EPI_OFF + (warp - 2) * EPI_STAGE_WARP, lane, xs, rp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(bar_tempty + 8 * acc);
                else mbar_arrive_cluster(tempty_leader + 8 * acc);
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    } else {
        // ------------------------------------------------ unpack warps: thread (r, h) expands half h (64 weights) of weight row r
        const int ut = threadIdx.x - (64 + EPI_THREADS);            // 0..255
        constexpr int CPT = 4 * BH / 256;                           // 16-byte chunks of a packed row per thread: 2 (MT = 1) or 1
        const int r = ut % BH, h = ut / BH, uw = ut >> 5;           // weight row, part of its K block; uw: unpack warp 0..7
        const int fb = wa.field_bits;
        const uint32_t psw = (uint32_t)((r >> 1) & 3), bsw = (uint32_t)(r & 7);
        const bool big_block = wa.f.block_shift >= 5;               // one block code covers (at least) a whole 16-byte chunk
        // The peer's warps signal the leader's `full` barrier with a 16-byte asynchronous copy into a spare slot of the leader's
        // shared memory that completes on that barrier: unlike a remote mbarrier arrive it does not hold the issuing warp up.
        const uint32_t sig_src = sbase + L::SIG_OFF + 16 * uw, sig_dst = mapa_u32(sbase + L::SIG_OFF + 128 + 16 * uw, 0);
        int stage = 0;
        uint32_t phase = 0;
        for (int t = pair; t < total && fail == 0; t += npairs) {
            const W4Tile tl = get_tile(t);
            const int ncol = tl.n0 + (int)rank * BH + r;                 // output column = weight row inside the matrix / expert
            const bool valid = ncol < a.N;
            const uint8_t* bcrow = wa.bcodes + (size_t)(tl.wbase + (int)rank * BH + r) * wa.bc_row;
            uint32_t field_next = 0;
            if (valid) field_next = fb == 8 ? bcrow[0] : fb == 16 ? *reinterpret_cast<const uint16_t*>(bcrow) : *reinterpret_cast<const uint32_t*>(bcrow);
            for (int kb = 0; kb < num_kb; ++kb) {
                const uint32_t field = field_next;
                if (valid && kb + 1 < num_kb) {
                    const uint8_t* pnext = bcrow + (size_t)(kb + 1) * (fb >> 3);
                    field_next = fb == 8 ? pnext[0] : fb == 16 ? *reinterpret_cast<const uint16_t*>(pnext) : *reinterpret_cast<const uint32_t*>(pnext);
                }
                int w = 0;                                   // one lane waits; the warp then agrees on the outcome
                if (lane == 0) w = mbar_wait(bar_loaded + 8 * stage, phase, abort_flag, a.wait_ns);
                __syncwarp();
                w = __shfl_sync(0xffffffffu, w, 0);
                if (w) { fail = (w == 1 && lane == 0) ? 6 : -1; break; }
                uint8_t* st = smem + stage * L::STAGE_BYTES;
                const uint8_t* prow = st + L::A_BYTES + L::B_BYTES + r * 64;
                uint8_t* brow = st + L::A_BYTES + r * 128;
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc) {
                    const int c = CPT * h + cc;                                // 16-byte chunk of the packed row: weights 32c .. 32c+31
                    uint4 pv = *reinterpret_cast<const uint4*>(prow + ((c ^ psw) << 4));
                    if (!valid) pv = make_uint4(0, 0, 0, 0);
                    const uint32_t ww[4] = {pv.x, pv.y, pv.z, pv.w};
                    uint32_t o[8];
                    if (big_block) {
                        const uint32_t code = (field >> (((32 * c) >> wa.f.block_shift) << wa.f.bc_shift)) & wa.f.bc_mask;
                        const uint32_t m = POW2 ? (1u << code) : fmt_mult(wa.f, code);
                        const uint32_t mlo = wa.f.mag_lo * m, mhi = wa.f.mag_hi * m;
#pragma unroll
                        for (int i = 0; i < 4; ++i) decode_word_pq(ww[i], mlo, mhi, o[2 * i], o[2 * i + 1]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int k8 = 8 * (4 * c + i);                            // first weight of the word inside the K block
                            const uint32_t code = (field >> ((k8 >> wa.f.block_shift) << wa.f.bc_shift)) & wa.f.bc_mask;
                            const uint32_t m = POW2 ? (1u << code) : fmt_mult(wa.f, code);
                            decode_word_pq(ww[i], wa.f.mag_lo * m, wa.f.mag_hi * m, o[2 * i], o[2 * i + 1]);
                        }
                    }
                    // words 4c, 4c+1 -> bytes 32c .. 32c+15 (16-byte chunk 2c); words 4c+2, 4c+3 -> chunk 2c + 1
                    *reinterpret_cast<uint4*>(brow + (((2 * c) ^ bsw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(brow + (((2 * c + 1) ^ bsw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> visible to the MMA's reads
                __syncwarp();
                if (lane == 0) {
                    if (leader) {
                        if (uw == 0) mbar_expect_tx(bar_full + 8 * stage, 16 * W4_UNPACK_WARPS);   // arrive + the peer's signal bytes
                        else mbar_arrive(bar_full + 8 * stage);
                    } else {
                        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(sig_dst), "r"(sig_src), "n"(16), "r"(full_leader + 8 * stage) : "memory");
                    }
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    }

    // status[0]: 1 producer / free stage, 2 MMA / free accumulator, 3 MMA / operands, 4 epilogue / accumulator,
    // 6 unpack warp / packed tile; status[1] CTA, status[2] thread
    if (fail > 0) {
        if (atomicCAS(a.status, 0, fail) == 0) {
            a.status[1] = blockIdx.x;
            a.status[2] = threadIdx.x;
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();
    tc_fence_after();
    if (warp == 1) tmem_dealloc2(tmem_base, TMEM_COLS);
}

// Host side: shape rules of the packed-weight kernel, tensor maps, launch.  rows_w = weight rows in total (N, or E * N).
static int run_w4(const int8_t* xq, int64_t a_rows, const uint32_t* codes, const uint8_t* bcodes, int64_t rows_w, const DevFormat& f,
                  GemmArgs& g, cudaStream_t st) {
    W4Args wa = {};
    wa.f = f;
    wa.bcodes = bcodes;
    wa.bc_row = (int)(g.K / (f.block * f.blocks_per_byte));
    wa.field_bits = (128 / f.block) * f.bc_bits;
    g.wait_ns = g_wait_limit_ns;
    if (g.epi == 3) {
        int rc3 = silu_lut_ptr(st, &g.silu_lut);
        if (rc3) return rc3;
    }
    wa.g = g;
    // Super tiles (two row tiles per expanded weight tile) where a segment usually has more than one row tile: a dense problem
    // of more than 256 rows, experts with more than 256 rows on average.
    const bool super = g.E == 0 ? g.M > 2 * BM : (int64_t)g.M > (int64_t)g.E * 2 * BM;
    const int bn = super ? W4SmemT<2>::BN : W4SmemT<1>::BN;
    CUtensorMap tmA, tmP;
    int rc = make_map_u8(&tmA, xq, a_rows, g.K, BK, BM, 128);
    if (rc) return rc;
    rc = make_map_u8(&tmP, codes, rows_w, g.K / 2, BK / 2, bn / 2, 64);
    if (rc) return rc;
    int pairs = sm_count() / 2;
    if (g.E == 0) {
        const int rows_tile = super ? 4 * BM : 2 * BM;
        const int64_t tiles = ((g.M + rows_tile - 1) / rows_tile) * (int64_t)((g.N + bn - 1) / bn);
        if (tiles < pairs) pairs = (int)tiles;
    }
    static bool configured[64] = {};
    const int dev = current_device();
    SCMX_REQUIRE(dev >= 0, SCMX_ECUDA, "no current CUDA device (ordinal 0..63)");
    if (!configured[dev]) {
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemm_w4_pair_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4SmemT<1>::TOTAL));
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemm_w4_pair_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4SmemT<1>::TOTAL));
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemm_w4_pair_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4SmemT<2>::TOTAL));
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemm_w4_pair_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4SmemT<2>::TOTAL));
        configured[dev] = true;
    }
    const dim3 grid(2 * pairs), block(W4_THREADS);
    cudaError_t e;
    if (super)
        e = f.pow2 ? launch_pdl(gemm_w4_pair_kernel<true, 2>, grid, block, (size_t)W4SmemT<2>::TOTAL, st, tmA, tmP, wa)
                   : launch_pdl(gemm_w4_pair_kernel<false, 2>, grid, block, (size_t)W4SmemT<2>::TOTAL, st, tmA, tmP, wa);
    else
        e = f.pow2 ? launch_pdl(gemm_w4_pair_kernel<true, 1>, grid, block, (size_t)W4SmemT<1>::TOTAL, st, tmA, tmP, wa)
                   : launch_pdl(gemm_w4_pair_kernel<false, 1>, grid, block, (size_t)W4SmemT<1>::TOTAL, st, tmA, tmP, wa);
    SCMX_PDL_OK("gemm_w4_pair_kernel", e);
    return SCMX_OK;
}

// Whether the packed-weight kernel covers a format and K: one aligned block-code field of 8, 16 or 32 bits per 128-wide K block.
static int w4_supported(const DevFormat& f, int64_t K) {
    if (f.block_shift < 0 || f.block > 128 || K % 128 != 0) return 0;
    const int bits = (128 / f.block) * f.bc_bits;
    return bits == 8 || bits == 16 || bits == 32;
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_w4_supported(const scmx_format* fmt, int64_t K) {
    DevFormat f;
    if (make_dev_format(fmt, &f)) return 0;
    return w4_supported(f, K);
}

extern "C" int scmx_mm_w4(const int8_t* xq, const uint32_t* codes, const uint8_t* bcodes, int64_t M, int64_t N, int64_t K,
                          const scmx_format* fmt, int epi, const float* xscale, const float* wscale, const uint16_t* res, void* out,
                          int32_t* status, void* stream) {
    int rc = check_common("mm_w4", N, K, epi, xscale, wscale, out, status);
    if (rc) return rc;
    DevFormat f;
    rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    SCMX_REQUIRE(w4_supported(f, K), SCMX_EFORMAT, "mm_w4: needs K %% 128 == 0 and 8, 16 or 32 block-code bits per 128 weights");
    SCMX_REQUIRE(M >= 0 && M < (1ll << 30), SCMX_EINVAL, "mm_w4: M=%lld out of range", (long long)M);
    SCMX_REQUIRE(epi != 2 || res, SCMX_EINVAL, "mm_w4: epi 2 needs res");
    SCMX_REQUIRE(codes && bcodes && ((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(codes)) & 15) == 0 &&
                     (!res || (reinterpret_cast<uintptr_t>(res) & 15) == 0) &&
                     (reinterpret_cast<uintptr_t>(bcodes) & 3) == 0,
                 SCMX_EINVAL, "mm_w4: xq, codes and res must be 16-byte aligned, bcodes 4-byte aligned");
    if (M == 0) return SCMX_OK;
    GemmArgs g = {};
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.epi = epi; g.xscale = xscale; g.wscale = wscale; g.res = res; g.out = out;
    g.status = status;
    return run_w4(xq, M, codes, bcodes, N, f, g, (cudaStream_t)stream);
}

extern "C" int scmx_moe_mm_w4(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                              const int32_t* off, int E, int64_t N, int64_t K, const scmx_format* fmt, int epi, const float* xscale,
                              void* out, int32_t* status, void* stream) {
    int rc = check_common("moe_mm_w4", N, K, epi, xscale, wscale, out, status);
    if (rc) return rc;
    DevFormat f;
    rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    SCMX_REQUIRE(w4_supported(f, K), SCMX_EFORMAT, "moe_mm_w4: needs K %% 128 == 0 and 8, 16 or 32 block-code bits per 128 weights");
    SCMX_REQUIRE(epi != 2, SCMX_EINVAL, "moe_mm_w4: epi must be 0, 1 or 3");
    SCMX_REQUIRE(E >= 1 && E <= W4_MAX_E && R >= 0 && R < (1ll << 30) && off, SCMX_EINVAL, "moe_mm_w4: bad E (1..%d) / R / offsets", W4_MAX_E);
    SCMX_REQUIRE((int64_t)E * N < (1ll << 31), SCMX_ELIMIT, "moe_mm_w4: E*N too large");
    SCMX_REQUIRE(codes && bcodes && ((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(codes)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(bcodes) & 3) == 0,
                 SCMX_EINVAL, "moe_mm_w4: xq and codes must be 16-byte aligned, bcodes 4-byte aligned");
    if (R == 0) return SCMX_OK;
    GemmArgs g = {};
    g.M = (int)R; g.N = (int)N; g.K = (int)K; g.epi = epi; g.xscale = xscale; g.wscale = wscale; g.out = out;
    g.off = off; g.E = E; g.e_begin = 0; g.e_end = E; g.status = status;
    return run_w4(xq, R, codes, bcodes, (int64_t)E * N, f, g, (cudaStream_t)stream);
}

extern "C" int scmx_moe_mm_w4_ret(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                                  const int32_t* off, int E, int64_t N, int64_t K, const scmx_format* fmt, const float* xscale,
                                  const int32_t* ret_rank, const int32_t* ret_row, int world, void* const* out_peers,
                                  int32_t* status, void* stream) {
    int rc = check_common("moe_mm_w4_ret", N, K, 1, xscale, wscale, out_peers, status);
    if (rc) return rc;
    DevFormat f;
    rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    SCMX_REQUIRE(w4_supported(f, K), SCMX_EFORMAT, "moe_mm_w4_ret: needs K %% 128 == 0 and 8, 16 or 32 block-code bits per 128 weights");
    SCMX_REQUIRE(E >= 1 && E <= W4_MAX_E && R >= 0 && R < (1ll << 30) && off, SCMX_EINVAL, "moe_mm_w4_ret: bad E (1..%d) / R / offsets", W4_MAX_E);
    SCMX_REQUIRE((int64_t)E * N < (1ll << 31), SCMX_ELIMIT, "moe_mm_w4_ret: E*N too large");
    SCMX_REQUIRE(ret_rank && ret_row && world >= 1 && world <= 8, SCMX_EINVAL, "moe_mm_w4_ret: return map / world (1..8)");
    SCMX_REQUIRE(codes && bcodes && ((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(codes)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(bcodes) & 3) == 0,
                 SCMX_EINVAL, "moe_mm_w4_ret: xq and codes must be 16-byte aligned, bcodes 4-byte aligned");
    if (R == 0) return SCMX_OK;
    GemmArgs g = {};
    g.M = (int)R; g.N = (int)N; g.K = (int)K; g.epi = 1; g.xscale = xscale; g.wscale = wscale; g.out = out_peers[0];
    g.off = off; g.E = E; g.e_begin = 0; g.e_end = E; g.status = status;
    g.ret_rank = ret_rank; g.ret_row = ret_row;
    for (int i = 0; i < 8; ++i) {
        g.peer_out[i] = i < world ? static_cast<uint16_t*>(out_peers[i]) : nullptr;
        SCMX_REQUIRE(i >= world || (g.peer_out[i] != nullptr && (reinterpret_cast<uintptr_t>(g.peer_out[i]) & 15) == 0), SCMX_EINVAL,
                     "moe_mm_w4_ret: return buffer of rank %d is NULL or not 16-byte aligned", i);
    }
    return run_w4(xq, R, codes, bcodes, (int64_t)E * N, f, g, (cudaStream_t)stream);
}
