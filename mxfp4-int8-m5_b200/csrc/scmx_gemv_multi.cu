// Streaming W4A8 decode GEMV over a LIST of independent jobs (y_i = epilogue(W_i x_i)) in one persistent launch.
//
// One CTA per SM, 544 threads.  The work of all jobs is cut into tiles of consecutive weight rows (up to 64 KB of packed
// codes each) that are dealt round-robin to the CTAs.  Warp 16 is the producer: one thread streams, tile after tile and
// without pausing at matrix boundaries, everything a tile needs into a ring of three shared-memory stages with untiled
// bulk copies (cp.async.bulk) that complete on the stage's mbarrier: packed codes, block codes, the row scales, the job
// record and the job's INT8 activation row.  Warps 0..15 are consumers: a warp owns 4 rows and one K split of the tile,
// expands the 4-bit codes from shared memory in registers and accumulates exact INT32 totals with DP4A:
//
//   P = prmt(LUT, w)            selector nibble = the code itself; its top bit (the sign) switches the byte permute to
//   Q = prmt(LUT, w ^ 0x8888)   "replicate the sign of the selected byte", and magnitudes have a clear top bit, so P holds the
//                               magnitudes of the positive codes (0 elsewhere) and Q those of the negative codes;
//   acc+ = dp4a(x, P, acc+);  acc- = dp4a(x, Q, acc-);  total = acc+ - acc-          (no negated copy of x, no sign select)
//
// with the block multiplier folded into the LUT by one integer multiply per block.  Row totals are reduced over the warp
// with 6 shuffles (4 values transposed while folding), K splits are added through shared-memory atomics (the last
// split to arrive finishes; nobody waits), and lanes 0 / 8 / 16 / 24 apply the GEMM's epilogue to one row each.
// Every mbarrier wait is bounded; a wait that runs out is reported through the status word and the kernel returns.
//
// Replaces the per-call GEMV launches of e2e/sc_decode.py:208-238 where many independent GEMVs are issued back to back
// (the reference's own timing protocol, e2e/tune_07.py:19-28, evaluates a batch of calls as one graph), and serves
// scmx_gemv for single large matrices.
#include "scmx_common.cuh"
#include "scmx_ptx.cuh"
#include "scmx_gemv_core.cuh"

namespace scmx {

constexpr int GM_CODES = 65536;            // packed codes per stage
constexpr int GM_BC = 2048;                // block codes per stage
constexpr int GM_WS = 256;                 // row scales per stage (64 rows)
constexpr int GM_JOB = 128;                // sizeof(scmx_gemv_job)
constexpr int GM_X = 8192;                 // INT8 activations (K <= 8192)
constexpr int GM_OFF_BC = GM_CODES, GM_OFF_WS = GM_OFF_BC + GM_BC, GM_OFF_JOB = GM_OFF_WS + GM_WS, GM_OFF_X = GM_OFF_JOB + GM_JOB;
constexpr int GM_STAGE = GM_OFF_X + GM_X;  // 76160 bytes
constexpr int GM_STAGES = 3;
constexpr int GM_NW = 16;                  // consumer warps
constexpr int GM_THREADS = 32 * (GM_NW + 1);
constexpr int GM_MAX_JOBS = 512;           // tile-start table in shared memory
constexpr int GM_TAIL = 4 * (GM_MAX_JOBS + 1) + 1280 + 8 * 2 * GM_STAGES + 16 + GM_JOB;
constexpr int GM_SMEM = GM_STAGES * GM_STAGE + GM_TAIL + 128;
static_assert(sizeof(scmx_gemv_job) == GM_JOB, "scmx_gemv_job must be 128 bytes");
static_assert(GM_SMEM <= 232448, "shared memory of the streaming GEMV exceeds 227 KB");
static_assert(GM_STAGE % 128 == 0, "stage size");

// plan[] slots of a planned job
enum { PL_TR = 0, PL_RG, PL_SK, PL_TILE0, PL_NTILES, PL_BCROW, PL_KW, PL_MAGIC, PL_TOTAL };
constexpr int PL_MAGIC_VALUE = 0x5C4D0001;

struct MultiArgs {
    const scmx_gemv_job* jobs;     // device array (n > 1), or null: `single` is the only job
    int n_jobs;
    int total_tiles;
    int32_t* status;
    uint64_t wait_ns;
    DevFormat f;
    scmx_gemv_job single;
};

__device__ __forceinline__ uint4 gm_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t gm_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t gm_lds8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// 8 codes of word w against activations xa (codes 0..3) and xb (codes 4..7): positive magnitudes into ap, negative into an.
__device__ __forceinline__ void word_pq(uint32_t w, uint32_t xa, uint32_t xb, uint32_t mlo, uint32_t mhi, int& ap, int& an) {
    const uint32_t wx = w ^ 0x88888888u;
    ap = dp4a_ss(xa, prmt(mlo, mhi, w), ap);
    an = dp4a_ss(xa, prmt(mlo, mhi, wx), an);
    ap = dp4a_ss(xb, prmt(mlo, mhi, w >> 16), ap);
    an = dp4a_ss(xb, prmt(mlo, mhi, wx >> 16), an);
}

// Block multiplier of block code `code`: a shift for power-of-two tables, else a lookup.
template <bool POW2>
__device__ __forceinline__ uint32_t gm_mult(const DevFormat& f, uint32_t code) {
    return POW2 ? (1u << code) : fmt_mult(f, code);
}

template <bool B32, bool POW2>
__global__ void __launch_bounds__(GM_THREADS, 1) gemv_multi_kernel(const __grid_constant__ MultiArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    // tail: barriers [2 * STAGES] | abort flag (16 B) | single job (128 B) | split-K sums [4][16][4] | split-K counters [4][16]
    //       | tile-start table [MAX_JOBS + 1]
    uint8_t* tail = smem + GM_STAGES * GM_STAGE;
    const uint32_t bar_full = smem_u32(tail), bar_empty = bar_full + 8 * GM_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * 2 * GM_STAGES);
    scmx_gemv_job* s_single = reinterpret_cast<scmx_gemv_job*>(tail + 8 * 2 * GM_STAGES + 16);
    int* s_part = reinterpret_cast<int*>(tail + 8 * 2 * GM_STAGES + 16 + GM_JOB);
    int* s_cnt = s_part + 256;
    int* s_tile0 = s_cnt + 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool multi = a.jobs != nullptr;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GM_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, GM_NW);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x < 320) s_part[threadIdx.x] = 0;
    // job records and their plans were written by the host long before this chain of kernels: readable before the wait
    if (multi) {
        for (int i = threadIdx.x; i <= a.n_jobs; i += GM_THREADS)
            s_tile0[i] = i < a.n_jobs ? a.jobs[i].plan[PL_TILE0] : a.total_tiles;
    } else {
        if (threadIdx.x < GM_JOB / 4)
            reinterpret_cast<uint32_t*>(s_single)[threadIdx.x] = reinterpret_cast<const uint32_t*>(&a.single)[threadIdx.x];
        if (threadIdx.x == 0) { s_tile0[0] = 0; s_tile0[1] = a.total_tiles; }
    }
    pdl_launch_dependents();
    __syncthreads();
    int fail = 0;

    if (warp == GM_NW) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            int stage = 0, d = 0, pending = 0;
            uint32_t phase = 0;
            bool waited = false;
            // activation copies of the first tiles are held back until the previous kernel of the stream has finished
            uint32_t x_dst[GM_STAGES], x_bar[GM_STAGES], x_len[GM_STAGES];
            const int8_t* x_src[GM_STAGES];
            for (int t = blockIdx.x; t < a.total_tiles; t += gridDim.x) {
                while (t >= s_tile0[d + 1]) ++d;
                const scmx_gemv_job* jp = multi ? a.jobs + d : &a.single;
                const int K = jp->K, N = jp->N, tr = jp->plan[PL_TR], bc_row = jp->plan[PL_BCROW];
                const uint8_t* codes = reinterpret_cast<const uint8_t*>(jp->codes);
                const uint8_t* bcodes = jp->bcodes;
                const float* wscale = jp->wscale;
                const int8_t* xq = jp->xq;
                if (int w = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, a.wait_ns)) { fail = w == 1 ? 1 : -1; break; }
                const int r0 = (t - s_tile0[d]) * tr;
                const int rows = min(tr, N - r0);
                const uint32_t dst = smem_u32(smem + stage * GM_STAGE), bar = bar_full + 8 * stage;
                const uint32_t nb_codes = (uint32_t)rows * (uint32_t)(K / 2), nb_bc = (uint32_t)rows * (uint32_t)bc_row;
                const uint32_t nb_ws = (uint32_t)rows * 4u, nb_job = multi ? (uint32_t)GM_JOB : 0u;
                mbar_expect_tx(bar, nb_codes + nb_bc + nb_ws + nb_job + (uint32_t)K);
                bulk_load(dst, codes + (size_t)r0 * (K / 2), nb_codes, bar);
                bulk_load(dst + GM_OFF_BC, bcodes + (size_t)r0 * bc_row, nb_bc, bar);
                bulk_load(dst + GM_OFF_WS, wscale + r0, nb_ws, bar);
                if (multi) bulk_load(dst + GM_OFF_JOB, jp, GM_JOB, bar);
                if (!waited && pending < GM_STAGES - 1) {
                    x_dst[pending] = dst + GM_OFF_X; x_bar[pending] = bar; x_len[pending] = (uint32_t)K; x_src[pending] = xq;
                    ++pending;
                } else {
                    if (!waited) {
                        pdl_wait();
                        waited = true;
                        for (int i = 0; i < pending; ++i) bulk_load(x_dst[i], x_src[i], x_len[i], x_bar[i]);
                    }
                    bulk_load(dst + GM_OFF_X, xq, (uint32_t)K, bar);
                }
                if (++stage == GM_STAGES) { stage = 0; phase ^= 1; }
            }
            if (!waited) {
                pdl_wait();
                for (int i = 0; i < pending; ++i) bulk_load(x_dst[i], x_src[i], x_len[i], x_bar[i]);
            }
        }
    } else {
        // ---------------------------------------------------------------- consumers
        pdl_wait();        // outputs, residuals and scales belong to the stream's earlier kernels
        int stage = 0, it = 0;
        uint32_t phase = 0;
        const int role_row = lane >> 3;            // lanes 0, 8, 16, 24 finish rows 0..3 of the warp's group
        const bool role = (lane & 7) == 0;
        for (int t = blockIdx.x; t < a.total_tiles; t += gridDim.x) {
            if (int w = mbar_wait(bar_full + 8 * stage, phase, abort_flag, a.wait_ns)) fail = w == 1 ? 2 : -1;
            if (fail) break;
            const uint8_t* st = smem + stage * GM_STAGE;
            const uint32_t st_s = smem_u32(st);
            const scmx_gemv_job* jp = multi ? reinterpret_cast<const scmx_gemv_job*>(st + GM_OFF_JOB) : s_single;
            const int K = jp->K, N = jp->N, epi = jp->epi;
            const int tr = jp->plan[PL_TR], rg = jp->plan[PL_RG], sk = jp->plan[PL_SK], kw = jp->plan[PL_KW];
            const int bc_row = jp->plan[PL_BCROW], row_bytes = K >> 1;
            const int r0t = (t - jp->plan[PL_TILE0]) * tr;
            const bool active = warp < rg * sk;
            const int rgi = active ? warp % rg : 0, ks = active ? warp / rg : 0;
            const int r0 = r0t + 4 * rgi;
            const bool rows_ok = active && r0 < N;
            // values the finishing lanes need, fetched early so that their latency hides behind the arithmetic
            float xs = 0.0f, wsr = 0.0f, resv = 0.0f;
            void* outp = jp->out;
            if (rows_ok && role) {
                if (epi != 0) xs = __ldg(jp->xscale);
                if (epi == 2) resv = bf16_to_f32(jp->res[r0 + role_row]);
                wsr = *reinterpret_cast<const float*>(st + GM_OFF_WS + 4 * (4 * rgi + role_row));
            }
            int tot[4] = {0, 0, 0, 0};
            if (rows_ok) {
                const int kbeg = ks * kw, kend = kbeg + kw;
                const uint32_t rows_s = st_s + (uint32_t)(4 * rgi) * (uint32_t)row_bytes;
                const uint32_t bc_s = st_s + GM_OFF_BC + (uint32_t)(4 * rgi) * (uint32_t)bc_row;
                int accp[4] = {0, 0, 0, 0}, accn[4] = {0, 0, 0, 0};
#pragma unroll 1
                for (int k0 = kbeg + lane * 32; k0 < kend; k0 += 1024) {
                    const uint4 xa = gm_lds128(st_s + GM_OFF_X + (uint32_t)k0);
                    const uint4 xb = gm_lds128(st_s + GM_OFF_X + (uint32_t)k0 + 16u);
                    const uint32_t x[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                    uint4 wv[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) wv[r] = gm_lds128(rows_s + (uint32_t)r * (uint32_t)row_bytes + (uint32_t)(k0 >> 1));
                    if (B32) {
                        // one block code per row for the lane's 32 codes
                        const int blk = k0 >> a.f.block_shift;
                        const uint32_t boff = (uint32_t)(blk >> a.f.pb_shift), bsh = (uint32_t)((blk & a.f.pb_mask) << a.f.bc_shift);
                        uint32_t code[4];
#pragma unroll
                        for (int r = 0; r < 4; ++r) code[r] = (gm_lds8(bc_s + (uint32_t)r * (uint32_t)bc_row + boff) >> bsh) & a.f.bc_mask;
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const uint32_t ww[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
                            if (POW2) {
                                // power-of-two multipliers: the block's sum with the plain table, shifted once (measured faster
                                // than scaling the table per block: 51.8 against 49.4 weights per clock per SM)
                                int bp = 0, bn = 0;
#pragma unroll
                                for (int j = 0; j < 4; ++j) word_pq(ww[j], x[2 * j], x[2 * j + 1], a.f.mag_lo, a.f.mag_hi, bp, bn);
                                accp[r] += (bp - bn) << code[r];
                            } else {
                                const uint32_t m = fmt_mult(a.f, code[r]);
                                const uint32_t mlo = a.f.mag_lo * m, mhi = a.f.mag_hi * m;     // per-byte products <= 127: no carries
#pragma unroll
                                for (int j = 0; j < 4; ++j) word_pq(ww[j], x[2 * j], x[2 * j + 1], mlo, mhi, accp[r], accn[r]);
                            }
                        }
                    } else {
                        // blocks of 8 or 16 codes: the block codes of the lane's 32 codes form one aligned bit field
                        const int nbits = (32 >> a.f.block_shift) << a.f.bc_shift;
                        const int bit0 = (k0 >> a.f.block_shift) << a.f.bc_shift;
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const uint32_t field = gm_lds32(bc_s + (uint32_t)r * (uint32_t)bc_row + (uint32_t)((bit0 >> 5) << 2)) >> (bit0 & 31);
                            const uint32_t ww[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t code = (field >> (((8 * j) >> a.f.block_shift) << a.f.bc_shift)) & a.f.bc_mask;
                                const uint32_t m = gm_mult<POW2>(a.f, code);
                                word_pq(ww[j], x[2 * j], x[2 * j + 1], a.f.mag_lo * m, a.f.mag_hi * m, accp[r], accn[r]);
                            }
                        }
                        (void)nbits;
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) tot[r] = accp[r] - accn[r];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * stage);       // this warp no longer reads the stage
            if (++stage == GM_STAGES) { stage = 0; phase ^= 1; }
            const int slot = it & 3;
            ++it;
            if (!active) continue;
            // sum over the warp: fold the 4 row totals while halving (6 shuffles); lane L ends with row 2*(L>>4&1) + (L>>3&1)
            const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0;
            int va = b4 ? tot[2] : tot[0], sa = b4 ? tot[0] : tot[2];
            int vb = b4 ? tot[3] : tot[1], sb = b4 ? tot[1] : tot[3];
            va += __shfl_xor_sync(0xffffffffu, sa, 16);
            vb += __shfl_xor_sync(0xffffffffu, sb, 16);
            int vc = b3 ? vb : va;
            const int sc = b3 ? va : vb;
            vc += __shfl_xor_sync(0xffffffffu, sc, 8);
            vc += __shfl_xor_sync(0xffffffffu, vc, 4);
            vc += __shfl_xor_sync(0xffffffffu, vc, 2);
            vc += __shfl_xor_sync(0xffffffffu, vc, 1);
            // (row index of lane L: bit 4 selects rows 2,3; bit 3 selects the odd row) = 2 * b4 + b3 = role_row for L = 0,8,16,24
            bool writer = true;
            if (sk > 1) {
                // add the K splits of the row group (exact integers) without a barrier: the last split to arrive finishes
                int* accq = s_part + (slot * 16 + rgi) * 4;
                if (role) atomicAdd(accq + role_row, vc);
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    __threadfence_block();
                    last = atomicAdd(s_cnt + slot * 16 + rgi, 1) == sk - 1;
                }
                writer = __shfl_sync(0xffffffffu, last, 0) != 0;
                if (writer) {
                    __threadfence_block();
                    if (role) vc = atomicExch(accq + role_row, 0);
                    if (lane == 0) atomicExch(s_cnt + slot * 16 + rgi, 0);
                }
            }
            if (!writer || !rows_ok) continue;
            const int row = r0 + role_row;
            if (epi == 0) {
                if (role) reinterpret_cast<int32_t*>(outp)[row] = vc;
                continue;
            }
            const float y = scale_acc(vc, xs, wsr);
            uint16_t* out = reinterpret_cast<uint16_t*>(outp);
            if (epi == 3) {
                const float yu = __shfl_down_sync(0xffffffffu, y, 16);      // rows 0,1 are gates; 2,3 the matching up rows
                if (role && role_row < 2) out[r0 / 2 + role_row] = f32_to_bf16(swiglu_bf16(y, yu));
            } else if (role) {
                out[row] = f32_to_bf16(epi == 2 ? __fadd_rn(resv, y) : y);
            }
        }
    }
    if (fail > 0 && a.status && atomicCAS(a.status, 0, 10 + fail) == 0) {
        a.status[1] = blockIdx.x;
        a.status[2] = threadIdx.x;
    }
    __syncthreads();
    if (*abort_flag) {      // give outstanding bulk copies time to land before the shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
}

// ---- host side --------------------------------------------------------------------------------------------------------------

// Tile geometry for a K: row groups rg (4 rows each) and K splits sk with rg * sk <= 16 consumer warps, rows * K / 2 <= 64 KB,
// every split a whole number of 32-code lane chunks; prefers more busy warps, then full 1024-code steps, then larger tiles.
static bool plan_tile(int64_t K, int* rg_out, int* sk_out) {
    int best_rg = 0, best_sk = 0;
    long best_score = -1;
    for (int sk = 1; sk <= GM_NW; ++sk) {
        if (K % sk != 0 || (K / sk) % 32 != 0) continue;
        int rg = GM_NW / sk;
        while (rg > 0 && (int64_t)rg * 4 * (K / 2) > GM_CODES) --rg;
        if (rg <= 0) continue;
        const int64_t kw = K / sk;
        const int full = kw % 1024 == 0 ? 1 : 0;
        // idle lanes in the last step of a split cost arithmetic slots; idle warps do not
        const int64_t steps = (kw + 1023) / 1024;
        const double lane_eff = (double)kw / (double)(steps * 1024);
        const long score = (long)(lane_eff * 1000.0) * 100000 + (long)(rg * sk) * 1000 + rg * (full + 1);
        if (score > best_score) { best_score = score; best_rg = rg; best_sk = sk; }
    }
    if (best_score < 0) return false;
    *rg_out = best_rg;
    *sk_out = best_sk;
    return true;
}

static int check_job(const scmx_gemv_job& j, const DevFormat& f, int i) {
    SCMX_REQUIRE(j.codes && j.bcodes && j.wscale && j.xq && j.out, SCMX_EINVAL, "gemv_multi: job %d has a NULL pointer", i);
    SCMX_REQUIRE(j.K > 0 && j.K % 128 == 0 && j.K <= GM_X, SCMX_EINVAL, "gemv_multi: job %d: K=%d must be a multiple of 128 up to %d", i, j.K, GM_X);
    SCMX_REQUIRE(j.N > 0 && j.N % 4 == 0, SCMX_EINVAL, "gemv_multi: job %d: N=%d must be a positive multiple of 4", i, j.N);
    SCMX_REQUIRE(j.epi >= 0 && j.epi <= 3, SCMX_EINVAL, "gemv_multi: job %d: epi=%d outside 0..3", i, j.epi);
    SCMX_REQUIRE(j.epi == 0 || j.xscale, SCMX_EINVAL, "gemv_multi: job %d: xscale is NULL", i);
    SCMX_REQUIRE(j.epi != 2 || j.res, SCMX_EINVAL, "gemv_multi: job %d: epi 2 needs res", i);
    SCMX_REQUIRE(f.block == 8 || f.block == 16 || f.block % 32 == 0, SCMX_EFORMAT, "gemv_multi: block=%d must be 8, 16 or a multiple of 32", f.block);
    SCMX_REQUIRE(f.block_shift >= 0, SCMX_EFORMAT, "gemv_multi: block=%d must be a power of two", f.block);
    SCMX_REQUIRE(j.K % (f.block * f.blocks_per_byte) == 0, SCMX_EINVAL, "gemv_multi: job %d: K=%d not a multiple of block*codes_per_byte", i, j.K);
    const int bc_row = j.K / (f.block * f.blocks_per_byte);
    SCMX_REQUIRE(bc_row % 4 == 0, SCMX_ELIMIT, "gemv_multi: job %d: %d block-code bytes per row (must be a multiple of 4)", i, bc_row);
    const uintptr_t al = reinterpret_cast<uintptr_t>(j.codes) | reinterpret_cast<uintptr_t>(j.bcodes) |
                         reinterpret_cast<uintptr_t>(j.wscale) | reinterpret_cast<uintptr_t>(j.xq);
    SCMX_REQUIRE((al & 15) == 0, SCMX_EINVAL, "gemv_multi: job %d: codes, bcodes, wscale and xq must be 16-byte aligned", i);
    return SCMX_OK;
}

int plan_jobs(scmx_gemv_job* jobs, int n, const DevFormat& f) {
    int tile0 = 0;
    for (int i = 0; i < n; ++i) {
        scmx_gemv_job& j = jobs[i];
        int rc = check_job(j, f, i);
        if (rc) return rc;
        int rg = 0, sk = 0;
        SCMX_REQUIRE(plan_tile(j.K, &rg, &sk), SCMX_ELIMIT, "gemv_multi: job %d: no tile shape for K=%d", i, j.K);
        const int bc_row = j.K / (f.block * f.blocks_per_byte);
        while (rg > 1 && (int64_t)rg * 4 * bc_row > GM_BC) --rg;
        SCMX_REQUIRE((int64_t)rg * 4 * bc_row <= GM_BC, SCMX_ELIMIT, "gemv_multi: job %d: block codes of 4 rows exceed %d bytes", i, GM_BC);
        const int tr = 4 * rg;
        j.plan[PL_TR] = tr; j.plan[PL_RG] = rg; j.plan[PL_SK] = sk; j.plan[PL_TILE0] = tile0;
        j.plan[PL_NTILES] = (j.N + tr - 1) / tr; j.plan[PL_BCROW] = bc_row; j.plan[PL_KW] = j.K / sk; j.plan[PL_MAGIC] = PL_MAGIC_VALUE;
        SCMX_REQUIRE((int64_t)tile0 + j.plan[PL_NTILES] < (1ll << 30), SCMX_ELIMIT, "gemv_multi: too many tiles");
        tile0 += j.plan[PL_NTILES];
    }
    for (int i = 0; i < n; ++i) jobs[i].plan[PL_TOTAL] = tile0;
    return SCMX_OK;
}

int launch_jobs(const scmx_gemv_job* jobs_host, const scmx_gemv_job* jobs_dev, int n, const DevFormat& f, int32_t* status, int pdl,
                cudaStream_t st) {
    MultiArgs a = {};
    a.jobs = n > 1 ? jobs_dev : nullptr;
    a.n_jobs = n;
    a.total_tiles = jobs_host[0].plan[PL_TOTAL];
    a.status = status;
    a.wait_ns = g_wait_limit_ns;
    a.f = f;
    a.single = jobs_host[0];
    const int n_sm = sm_count();
    const int grid = a.total_tiles < n_sm ? a.total_tiles : n_sm;
    const bool b32 = f.block % 32 == 0, pow2 = f.pow2 != 0;
    static bool configured[64] = {};
    const int dev = current_device();
    SCMX_REQUIRE(dev >= 0, SCMX_ECUDA, "gemv_multi: no current CUDA device (ordinal 0..63)");
    if (!configured[dev]) {
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemv_multi_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemv_multi_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemv_multi_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemv_multi_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
        configured[dev] = true;
    }
    cudaError_t e;
    if (b32) e = pow2 ? launch_pdl_opt(pdl, gemv_multi_kernel<true, true>, dim3(grid), dim3(GM_THREADS), (size_t)GM_SMEM, st, a)
                      : launch_pdl_opt(pdl, gemv_multi_kernel<true, false>, dim3(grid), dim3(GM_THREADS), (size_t)GM_SMEM, st, a);
    else e = pow2 ? launch_pdl_opt(pdl, gemv_multi_kernel<false, true>, dim3(grid), dim3(GM_THREADS), (size_t)GM_SMEM, st, a)
                  : launch_pdl_opt(pdl, gemv_multi_kernel<false, false>, dim3(grid), dim3(GM_THREADS), (size_t)GM_SMEM, st, a);
    SCMX_PDL_OK("gemv_multi_kernel", e);
    return SCMX_OK;
}

// One dense GEMV through the streaming kernel (called by scmx_gemv); SCMX_ELIMIT = the shape does not fit it.
int gemv_stream_single(const int8_t* xq, const float* xscale, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                       int64_t N, int64_t K, const DevFormat& f, int epi, const uint16_t* res, void* out, int pdl, cudaStream_t st) {
    scmx_gemv_job j = {};
    j.codes = codes; j.bcodes = bcodes; j.wscale = wscale; j.xq = xq; j.xscale = xscale; j.res = res; j.out = out;
    j.N = (int32_t)N; j.K = (int32_t)K; j.epi = epi;
    int rc = plan_jobs(&j, 1, f);
    if (rc) return rc;
    return launch_jobs(&j, nullptr, 1, f, device_status_word(), pdl, st);
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_gemv_multi_plan(scmx_gemv_job* jobs, int n, const scmx_format* fmt) {
    SCMX_REQUIRE(jobs != nullptr && n >= 1 && n <= GM_MAX_JOBS, SCMX_EINVAL, "gemv_multi_plan: n=%d (1..%d jobs)", n, GM_MAX_JOBS);
    DevFormat f;
    int rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    return plan_jobs(jobs, n, f);
}

extern "C" int scmx_gemv_multi(const scmx_gemv_job* jobs_host, const scmx_gemv_job* jobs_dev, int n, const scmx_format* fmt,
                               int32_t* status, int pdl, void* stream) {
    SCMX_REQUIRE(jobs_host != nullptr && n >= 1 && n <= GM_MAX_JOBS, SCMX_EINVAL, "gemv_multi: n=%d (1..%d jobs)", n, GM_MAX_JOBS);
    SCMX_REQUIRE(n == 1 || (jobs_dev != nullptr && (reinterpret_cast<uintptr_t>(jobs_dev) & 15) == 0), SCMX_EINVAL,
                 "gemv_multi: the device copy of the job list is NULL or not 16-byte aligned");
    SCMX_REQUIRE(status != nullptr, SCMX_EINVAL, "gemv_multi: status is NULL");
    DevFormat f;
    int rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    int tiles = 0;
    for (int i = 0; i < n; ++i) {
        SCMX_REQUIRE(jobs_host[i].plan[PL_MAGIC] == PL_MAGIC_VALUE && jobs_host[i].plan[PL_TILE0] == tiles, SCMX_EINVAL,
                     "gemv_multi: job %d was not planned (call scmx_gemv_multi_plan on the list first)", i);
        rc = check_job(jobs_host[i], f, i);
        if (rc) return rc;
        tiles += jobs_host[i].plan[PL_NTILES];
    }
    SCMX_REQUIRE(tiles == jobs_host[0].plan[PL_TOTAL], SCMX_EINVAL, "gemv_multi: the plan does not match the list");
    return launch_jobs(jobs_host, jobs_dev, n, f, status, pdl, (cudaStream_t)stream);
}
