// Batch-1 W4A8 decode GEMV reading the packed 4-bit codes directly.  HBM-bound: no tensor cores.
//
// A warp owns 4 consecutive output rows and a slice of K.  Per step a lane streams 16 bytes (32 codes) of each of
// its rows with one 128-bit load; all loads of a warp (4 rows x STEPS steps) are issued before any is consumed so
// that enough bytes are in flight to cover DRAM latency.  Codes are expanded in registers: a byte permute looks up
// the magnitudes of four codes at once, a second byte permute picks x or -x per code according to the sign bit,
// and DP4A accumulates; the per-block integer multiplier is applied to the block sum.  Lane totals are exact INT32
// and are reduced with shuffles, across K-splits through shared memory.  The epilogue is the GEMM's
// (scale, + residual, SwiGLU), so GEMV and GEMM produce the same bits.
//
// With programmatic dependent launch the weight loads are issued before griddepcontrol.wait: they do not depend on
// the previous kernel, so they overlap its tail; activations, scales and expert ids are read after the wait.
#include "scmx_common.cuh"
#include "scmx_ptx.cuh"
#include "scmx_gemv_core.cuh"

namespace scmx {

struct GemvArgs {
    const int8_t* xq;
    const float* xscale;
    const uint32_t* codes;
    const uint8_t* bcodes;
    const float* wscale;
    const uint16_t* res;
    const int32_t* eidx;
    void* out;
    int N, K, epi, n_routed, shared, xstride;
    int sk;            // K splits (warps per row group)
    int rg;            // row groups per CTA
    int bc_row_bytes;
    const uint16_t* xbf;   // prologue forms: bf16 input row(s) [K] instead of xq / xscale
    const uint16_t* nw;    // RMSNorm weights (prologue 2)
    float eps;
    DevFormat f;
};

// sum over the 8 codes of word w of (+-x) * magnitude: 11 instructions
__device__ __forceinline__ int word_dot(uint32_t w, uint32_t x0, uint32_t xn0, uint32_t x1, uint32_t xn1, uint32_t mlo, uint32_t mhi,
                                        int acc) {
    const uint32_t sel = w & 0x77777777u;
    const uint32_t ssel = ((w >> 1) & 0x44444444u) | 0x32103210u;
    acc = dp4a_ss(prmt(x0, xn0, ssel), prmt(mlo, mhi, sel), acc);
    return dp4a_ss(prmt(x1, xn1, ssel >> 16), prmt(mlo, mhi, sel >> 16), acc);
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// PRO 0: INT8 input row and its scale are given.  PRO 1 / 2: the input is a bf16 row; every CTA first computes the
// per-token INT8 row (PRO 2: of its RMSNorm) in shared memory with the arithmetic of the row kernels (act_quant,
// rmsnorm_quant), after the weight loads are in flight, so the separate kernel and its launch disappear from the chain.
// Replaces the PRO 1 / PRO 2 prologues of e2e/sc_decode.py:50-65.
constexpr int GEMV_PRO_MAXK = 8192;

template <int PRO>
__device__ __forceinline__ float gemv_prologue(const GemvArgs& a, int slot, int8_t* xq_s, uint4* xn_s, float* red, double* dred) {
    const int K = a.K, nv = K / 8, nt = blockDim.x;
    const uint4* xrow = reinterpret_cast<const uint4*>(a.xbf + (size_t)slot * a.xstride * K);
    float amax = 0.0f;
    double ss = 0.0;
    for (int v = threadIdx.x; v < nv; v += nt) {
        const uint4 r = xrow[v];
        xn_s[v] = r;
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f0 = __uint_as_float(w[j] << 16), f1 = __uint_as_float(w[j] & 0xFFFF0000u);
            if (PRO == 2) ss += (double)f0 * (double)f0 + (double)f1 * (double)f1;
            else amax = fmaxf(amax, fmaxf(fabsf(f0), fabsf(f1)));
        }
    }
    if (PRO == 2) {
        ss = block_sum(ss, dred);
        const float inv = rms_inverse(ss, K, a.eps);
        const uint4* nw4 = reinterpret_cast<const uint4*>(a.nw);
        for (int v = threadIdx.x; v < nv; v += nt) {       // the vectors this thread staged itself
            const uint4 r = xn_s[v], wv = nw4[v];
            const uint32_t x[4] = {r.x, r.y, r.z, r.w}, w[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float f0 = rbf(__fmul_rn(__uint_as_float(w[j] << 16), rbf(__fmul_rn(__uint_as_float(x[j] << 16), inv))));
                const float f1 = rbf(__fmul_rn(__uint_as_float(w[j] & 0xFFFF0000u), rbf(__fmul_rn(__uint_as_float(x[j] & 0xFFFF0000u), inv))));
                amax = fmaxf(amax, fmaxf(fabsf(f0), fabsf(f1)));
                o[j] = (__float_as_uint(f0) >> 16) | (__float_as_uint(f1) & 0xFFFF0000u);
            }
            xn_s[v] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
    for (int v = threadIdx.x; v < nv; v += nt) {
        const uint4 r = xn_s[v];
        const uint32_t x[4] = {r.x, r.y, r.z, r.w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[2 * j] = __uint_as_float(x[j] << 16);
            f[2 * j + 1] = __uint_as_float(x[j] & 0xFFFF0000u);
        }
        reinterpret_cast<uint2*>(xq_s)[v] = make_uint2(quant4(f[0], f[1], f[2], f[3], qi), quant4(f[4], f[5], f[6], f[7], qi));
    }
    __syncthreads();
    return s;
}

template <int STEPS, bool B32, int PRO>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvArgs a) {
    __shared__ int part[8 * 4];
    __shared__ __align__(16) int8_t xq_s[PRO ? GEMV_PRO_MAXK : 16];
    __shared__ __align__(16) uint4 xn_s[PRO ? GEMV_PRO_MAXK / 8 : 1];
    __shared__ float red[33];
    __shared__ double dred[33];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int ks = wid % a.sk, rgi = wid / a.sk;
    const int n0 = (blockIdx.x * a.rg + rgi) * 4;
    const int slot = blockIdx.y;
    const bool rows_ok = n0 < a.N;
    const int K = a.K, wpr = K / 8;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int ex = 0;
    if (a.eidx) {   // expert ids come from the previous kernel: wait before anything else
        asm volatile("griddepcontrol.wait;" ::: "memory");
        ex = (a.shared >= 0 && slot == a.n_routed) ? a.shared : a.eidx[slot];
    }
    const uint32_t* codes = a.codes + (size_t)ex * a.N * wpr;
    const uint8_t* bcodes = a.bcodes + (size_t)ex * a.N * a.bc_row_bytes;

    uint4 w[STEPS][4];
    uint32_t bc[STEPS][4];
    int k0s[STEPS];
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
        const int k0 = ((ks + s * a.sk) * 32 + lane) * 32;
        k0s[s] = (rows_ok && k0 < K) ? k0 : -1;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            w[s][r] = make_uint4(0, 0, 0, 0);
            bc[s][r] = 0;
            if (k0s[s] >= 0) {
                w[s][r] = ldg_stream(reinterpret_cast<const uint4*>(codes + (size_t)(n0 + r) * wpr + k0 / 8));
                const uint8_t* rb = bcodes + (size_t)(n0 + r) * a.bc_row_bytes;
                if (B32) {
                    bc[s][r] = rb[block_of(a.f, k0) >> a.f.pb_shift];
                } else {
                    // the lane's 32 codes span 32/block blocks whose codes fit one aligned 32-bit field
                    const int bit0 = (k0 >> a.f.block_shift) << a.f.bc_shift;
                    uint32_t v = 0;
                    const int nbytes = (((32 >> a.f.block_shift) << a.f.bc_shift) + 7) / 8;
                    for (int i = 0; i < nbytes; ++i) v |= (uint32_t)rb[bit0 / 8 + i] << (8 * i);
                    bc[s][r] = v >> (bit0 % 8);
                }
            }
        }
    }
    if (!a.eidx) asm volatile("griddepcontrol.wait;" ::: "memory");

    float xs_pro = 0.0f;
    if (PRO) xs_pro = gemv_prologue<PRO>(a, slot, xq_s, xn_s, red, dred);
    const int8_t* xq = PRO ? xq_s : a.xq + (size_t)slot * a.xstride * K;
    int tot[4] = {0, 0, 0, 0};
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
        if (k0s[s] < 0) continue;
        const uint4 xa = *reinterpret_cast<const uint4*>(xq + k0s[s]);
        const uint4 xb = *reinterpret_cast<const uint4*>(xq + k0s[s] + 16);
        const uint32_t x[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        uint32_t xn[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) xn[j] = neg4(x[j]);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t ww[4] = {w[s][r].x, w[s][r].y, w[s][r].z, w[s][r].w};
            if (B32) {
                const int blk = block_of(a.f, k0s[s]);
                const uint32_t code = (bc[s][r] >> ((blk & a.f.pb_mask) << a.f.bc_shift)) & a.f.bc_mask;
                int bs = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t sel = ww[j] & 0x77777777u;
                    const uint32_t ssel = ((ww[j] >> 1) & 0x44444444u) | 0x32103210u;
                    bs = __dp4a((int)__byte_perm(x[2 * j], xn[2 * j], ssel), (int)__byte_perm(a.f.mag_lo, a.f.mag_hi, sel), bs);
                    bs = __dp4a((int)__byte_perm(x[2 * j + 1], xn[2 * j + 1], ssel >> 16),
                                (int)__byte_perm(a.f.mag_lo, a.f.mag_hi, sel >> 16), bs);
                }
                tot[r] += a.f.pow2 ? (bs << code) : bs * (int)fmt_mult(a.f, code);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int bi = (8 * j) >> a.f.block_shift;   // block index inside the lane's 32 codes
                    const uint32_t code = (bc[s][r] >> (bi << a.f.bc_shift)) & a.f.bc_mask;
                    const uint32_t sel = ww[j] & 0x77777777u;
                    const uint32_t ssel = ((ww[j] >> 1) & 0x44444444u) | 0x32103210u;
                    int bs = __dp4a((int)__byte_perm(x[2 * j], xn[2 * j], ssel), (int)__byte_perm(a.f.mag_lo, a.f.mag_hi, sel), 0);
                    bs = __dp4a((int)__byte_perm(x[2 * j + 1], xn[2 * j + 1], ssel >> 16),
                                (int)__byte_perm(a.f.mag_lo, a.f.mag_hi, sel >> 16), bs);
                    tot[r] += bs * (int)fmt_mult(a.f, code);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) tot[r] = warp_sum(tot[r]);
    if (a.sk > 1) {
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < 4; ++r) part[wid * 4 + r] = tot[r];
        }
        __syncthreads();
        if (ks != 0) return;
        for (int j = 1; j < a.sk; ++j) {
#pragma unroll
            for (int r = 0; r < 4; ++r) tot[r] += part[(wid + j) * 4 + r];
        }
    }
    if (lane != 0 || !rows_ok) return;
    const float* ws = a.wscale + (size_t)ex * a.N + n0;
    if (a.epi == 0) {
        int32_t* o = reinterpret_cast<int32_t*>(a.out) + (size_t)slot * a.N + n0;
#pragma unroll
        for (int r = 0; r < 4; ++r) o[r] = tot[r];
        return;
    }
    const float xs = PRO ? xs_pro : a.xscale[(size_t)slot * a.xstride];
    float y[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) y[r] = scale_acc(tot[r], xs, ws[r]);
    uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
    if (a.epi == 1) {
        uint16_t* o = out + (size_t)slot * a.N + n0;
#pragma unroll
        for (int r = 0; r < 4; ++r) o[r] = f32_to_bf16(y[r]);
    } else if (a.epi == 2) {
        uint16_t* o = out + (size_t)slot * a.N + n0;
#pragma unroll
        for (int r = 0; r < 4; ++r) o[r] = f32_to_bf16(__fadd_rn(bf16_to_f32(a.res[n0 + r]), y[r]));
    } else {
        uint16_t* o = out + (size_t)slot * (a.N / 2) + n0 / 2;
        o[0] = f32_to_bf16(swiglu_bf16(y[0], y[2]));
        o[1] = f32_to_bf16(swiglu_bf16(y[1], y[3]));
    }
}

// ---- streaming variant for dense GEMVs ------------------------------------------------------------------------------------
// A persistent CTA (one per SM, 544 threads) walks over tiles of TR consecutive weight rows.  The rows of a tile are
// contiguous in the packed layout, so one thread streams each tile into a shared-memory ring with two untiled bulk copies
// (codes, block codes) that complete on an mbarrier; sixteen consumer warps expand and accumulate from shared memory
// (warp = 4 rows x one K split) and release the stage through a second mbarrier.  Copies run STAGES tiles ahead of the
// arithmetic, and since weights do not depend on the previous kernel they start before griddepcontrol.wait: with one CTA
// of < 112 KB per SM the next GEMV of a chain is already resident and filling its ring while this one finishes.
constexpr int SG_STAGE_BYTES = 65536;      // packed codes per stage
constexpr int SG_BC_BYTES = 2048;          // block codes per stage
constexpr int SG_X_BYTES = 8192;           // INT8 activations (K <= 8192)
constexpr int SG_STAGES = 3;
constexpr int SG_NW = 16;                  // consumer warps
constexpr int SG_THREADS = 32 * (SG_NW + 1);   // consumer warps + 1 producer warp

struct StreamArgs {
    GemvArgs g;
    int tr;            // rows per tile (4, 8, 16, 32 or 64)
    int n_tiles;
    int mode;          // 0 normal; 1 = measurement aid: stream the tiles but skip the arithmetic
    int32_t* status;
};

template <bool B32>
__global__ void __launch_bounds__(SG_THREADS, 1) gemv_stream_kernel(const StreamArgs sa) {
    extern __shared__ uint8_t smem_raw[];
    const GemvArgs& a = sa.g;
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);     // stays a shared-space pointer
    // layout: [STAGES][codes 64 KB][bcodes 2 KB] | x (K bytes) | split-K sums [4][16][4] | split-K counters [4][16] |
    //         barriers | abort flag
    uint8_t* s_x = smem + SG_STAGES * (SG_STAGE_BYTES + SG_BC_BYTES);
    int* s_part = reinterpret_cast<int*>(s_x + SG_X_BYTES);
    int* s_cnt = s_part + 256;
    const uint32_t bar_full = smem_u32(s_cnt + 64), bar_empty = bar_full + 8 * SG_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(s_cnt + 64 + 4 * SG_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = a.K, row_bytes = K / 2, bc_row = a.bc_row_bytes;
    if (threadIdx.x == 0) {
        for (int s = 0; s < SG_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, SG_NW);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x < 320) s_part[threadIdx.x] = 0;      // split-K sums and counters
    pdl_launch_dependents();
    __syncthreads();
    int fail = 0;
    if (warp == SG_NW) {
        // ---- producer: weights only, so it does not wait for the previous kernel
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = blockIdx.x; t < sa.n_tiles; t += gridDim.x) {
                if (int w = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag)) { fail = w == 1 ? 1 : -1; break; }
                const int r0 = t * sa.tr;
                const int rows = min(sa.tr, a.N - r0);
                const uint32_t dst = smem_u32(smem + stage * (SG_STAGE_BYTES + SG_BC_BYTES));
                const uint32_t nb_codes = (uint32_t)rows * row_bytes, nb_bc = (uint32_t)rows * bc_row;
                mbar_expect_tx(bar_full + 8 * stage, nb_codes + nb_bc);
                bulk_load(dst, reinterpret_cast<const uint8_t*>(a.codes) + (size_t)r0 * row_bytes, nb_codes, bar_full + 8 * stage);
                bulk_load(dst + SG_STAGE_BYTES, a.bcodes + (size_t)r0 * bc_row, nb_bc, bar_full + 8 * stage);
                if (++stage == SG_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        // ---- consumers: activations come from the previous kernel
        pdl_wait();
        for (int i = threadIdx.x; i < K / 16; i += 32 * SG_NW)
            reinterpret_cast<uint4*>(s_x)[i] = reinterpret_cast<const uint4*>(a.xq)[i];
        asm volatile("bar.sync 1, %0;" ::"n"(32 * SG_NW) : "memory");
        const int rg = sa.tr / 4;                 // row groups per tile
        const int sk = SG_NW / rg;                // K splits per row group
        const int rgi = warp % rg, ks = warp / rg;
        const int kbeg = ks * (K / sk), kend = kbeg + K / sk;
        const float xs = a.epi != 0 ? a.xscale[0] : 0.0f;
        const uint32_t mlo = a.f.mag_lo, mhi = a.f.mag_hi;
        // A lane visits the same K offsets in every tile.  When its K range is at most two steps of 1024 codes the
        // activations (and their negations) for those offsets stay in registers for the whole kernel.
        const bool xcache = (kend - kbeg) <= 2048;
        uint32_t xr[2][8], xnr[2][8];
#pragma unroll
        for (int sidx = 0; sidx < 2; ++sidx) {
            const int k0 = kbeg + lane * 32 + sidx * 1024;
            const bool ok = xcache && k0 < kend;
            const uint4 xa = ok ? *reinterpret_cast<const uint4*>(s_x + k0) : make_uint4(0, 0, 0, 0);
            const uint4 xb = ok ? *reinterpret_cast<const uint4*>(s_x + k0 + 16) : make_uint4(0, 0, 0, 0);
            const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) { xr[sidx][j] = xv[j]; xnr[sidx][j] = neg4(xv[j]); }
        }
        // block-code byte offset and bit shift of the lane's (up to two cached) K offsets: the same for every row and tile
        uint32_t bc_off[2], bc_sh[2];
#pragma unroll
        for (int sidx = 0; sidx < 2; ++sidx) {
            const int blk = block_of(a.f, kbeg + lane * 32 + sidx * 1024);
            bc_off[sidx] = (uint32_t)(blk >> a.f.pb_shift);
            bc_sh[sidx] = (uint32_t)((blk & a.f.pb_mask) << a.f.bc_shift);
        }
        const uint32_t row_off = (uint32_t)(4 * rgi) * (uint32_t)row_bytes, rb_off = SG_STAGE_BYTES + (uint32_t)(4 * rgi) * (uint32_t)bc_row;
        int stage = 0, it = 0;
        uint32_t phase = 0;
        for (int t = blockIdx.x; t < sa.n_tiles; t += gridDim.x) {
            if (int w = mbar_wait(bar_full + 8 * stage, phase, abort_flag)) { fail = w == 1 ? 2 : -1; }
            if (fail) break;
            const uint8_t* st = smem + stage * (SG_STAGE_BYTES + SG_BC_BYTES);
            const uint32_t st_s = smem_u32(st);
            const int r0 = t * sa.tr + 4 * rgi;      // first of this warp's 4 rows
            const bool rows_ok = r0 < a.N;
            int tot[4] = {0, 0, 0, 0};
            if (rows_ok) {
#pragma unroll 2
                for (int sidx = 0; sidx < 32; ++sidx) {
                    const int k0 = kbeg + lane * 32 + sidx * 1024;
                    if (k0 >= kend) break;
                    uint32_t x[8], xn[8];
                    if (xcache) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) { x[j] = xr[sidx & 1][j]; xn[j] = xnr[sidx & 1][j]; }
                    } else {
                        const uint4 xa = *reinterpret_cast<const uint4*>(s_x + k0);
                        const uint4 xb = *reinterpret_cast<const uint4*>(s_x + k0 + 16);
                        const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) { x[j] = xv[j]; xn[j] = neg4(xv[j]); }
                    }
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint32_t row_s = st_s + row_off + (uint32_t)r * (uint32_t)row_bytes;
                        const uint4 wv = lds128(row_s + (uint32_t)(k0 >> 1));
                        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
                        if (sa.mode == 1) { tot[r] += (int)(ww[0] ^ ww[1] ^ ww[2] ^ ww[3] ^ x[r]); continue; }
                        const uint32_t rb_s = st_s + rb_off + (uint32_t)r * (uint32_t)bc_row;
                        const uint8_t* rb = st + SG_STAGE_BYTES + (size_t)(4 * rgi + r) * bc_row;
                        if (B32) {
                            uint32_t code;
                            if (xcache) {
                                code = (lds8(rb_s + bc_off[sidx & 1]) >> bc_sh[sidx & 1]) & a.f.bc_mask;
                            } else {
                                const int blk = block_of(a.f, k0);
                                code = (lds8(rb_s + (uint32_t)(blk >> a.f.pb_shift)) >> ((blk & a.f.pb_mask) << a.f.bc_shift)) & a.f.bc_mask;
                            }
                            int bs = 0;
#pragma unroll
                            for (int j = 0; j < 4; ++j) bs = word_dot(ww[j], x[2 * j], xn[2 * j], x[2 * j + 1], xn[2 * j + 1], mlo, mhi, bs);
                            tot[r] += a.f.pow2 ? (bs << code) : bs * (int)fmt_mult(a.f, code);
                        } else {
                            const int bit0 = (k0 >> a.f.block_shift) << a.f.bc_shift;
                            const int nbytes = (((32 >> a.f.block_shift) << a.f.bc_shift) + 7) / 8;
                            uint32_t bcv = 0;
                            for (int i = 0; i < nbytes; ++i) bcv |= (uint32_t)rb[bit0 / 8 + i] << (8 * i);
                            bcv >>= (bit0 % 8);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int bi = (8 * j) >> a.f.block_shift;
                                const uint32_t code = (bcv >> (bi << a.f.bc_shift)) & a.f.bc_mask;
                                const uint32_t sel = ww[j] & 0x77777777u;
                                const uint32_t ssel = ((ww[j] >> 1) & 0x44444444u) | 0x32103210u;
                                int bs = __dp4a((int)__byte_perm(x[2 * j], xn[2 * j], ssel), (int)__byte_perm(a.f.mag_lo, a.f.mag_hi, sel), 0);
                                bs = __dp4a((int)__byte_perm(x[2 * j + 1], xn[2 * j + 1], ssel >> 16),
                                            (int)__byte_perm(a.f.mag_lo, a.f.mag_hi, sel >> 16), bs);
                                tot[r] += bs * (int)fmt_mult(a.f, code);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * stage);       // this warp no longer reads the stage
            if (++stage == SG_STAGES) { stage = 0; phase ^= 1; }
#pragma unroll
            for (int r = 0; r < 4; ++r) tot[r] = warp_sum(tot[r]);
            bool writer = lane == 0;
            if (sk > 1 && lane == 0) {
                // add the K splits of a row group (exact integers) without a barrier: the last split to arrive finishes
                int* accp = s_part + ((it & 3) * 16 + rgi) * 4;
#pragma unroll
                for (int r = 0; r < 4; ++r) atomicAdd(accp + r, tot[r]);
                __threadfence_block();
                const int c = atomicAdd(s_cnt + (it & 3) * 16 + rgi, 1);
                writer = c == sk - 1;
                if (writer) {
                    __threadfence_block();
#pragma unroll
                    for (int r = 0; r < 4; ++r) tot[r] = atomicExch(accp + r, 0);
                    atomicExch(s_cnt + (it & 3) * 16 + rgi, 0);
                }
            }
            ++it;
            if (writer && rows_ok) {
                const float* ws = a.wscale + r0;
                if (a.epi == 0) {
                    int32_t* o = reinterpret_cast<int32_t*>(a.out) + r0;
#pragma unroll
                    for (int r = 0; r < 4; ++r) o[r] = tot[r];
                } else {
                    float y[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) y[r] = scale_acc(tot[r], xs, ws[r]);
                    uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
                    if (a.epi == 1) {
#pragma unroll
                        for (int r = 0; r < 4; ++r) out[r0 + r] = f32_to_bf16(y[r]);
                    } else if (a.epi == 2) {
#pragma unroll
                        for (int r = 0; r < 4; ++r) out[r0 + r] = f32_to_bf16(__fadd_rn(bf16_to_f32(a.res[r0 + r]), y[r]));
                    } else {
                        out[r0 / 2] = f32_to_bf16(swiglu_bf16(y[0], y[2]));
                        out[r0 / 2 + 1] = f32_to_bf16(swiglu_bf16(y[1], y[3]));
                    }
                }
            }
        }
    }
    if (fail > 0 && sa.status && atomicCAS(sa.status, 0, 10 + fail) == 0) {
        sa.status[1] = blockIdx.x;
        sa.status[2] = threadIdx.x;
    }
    __syncthreads();
    if (*abort_flag) {      // give outstanding bulk copies time to land before the shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
}

template <int STEPS, bool B32>
static cudaError_t launch_gemv(const GemvArgs& a, dim3 grid, int threads, int pdl, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (a.xbf != nullptr) {
        if (a.nw != nullptr) return cudaLaunchKernelEx(&cfg, gemv_kernel<STEPS, B32, 2>, a);
        return cudaLaunchKernelEx(&cfg, gemv_kernel<STEPS, B32, 1>, a);
    }
    return cudaLaunchKernelEx(&cfg, gemv_kernel<STEPS, B32, 0>, a);
}

}  // namespace scmx

using namespace scmx;

static int g_gemv_stream = 1;
extern "C" int scmx_set_gemv_stream(int enable) {
    g_gemv_stream = enable;
    return SCMX_OK;
}

static int gemv_impl(const int8_t* xq, const float* xscale, const uint16_t* xbf, const uint16_t* nw, float eps, const uint32_t* codes,
                     const uint8_t* bcodes, const float* wscale, int64_t N, int64_t K, const scmx_format* fmt, int epi,
                     const uint16_t* res, const int32_t* eidx, int n_routed, int shared, int xstride, void* out, int pdl,
                     void* stream) {
    GemvArgs a;
    int rc = make_dev_format(fmt, &a.f);
    if (rc) return rc;
    a.xbf = xbf; a.nw = nw; a.eps = eps;
    if (xbf != nullptr) {
        SCMX_REQUIRE(K <= GEMV_PRO_MAXK, SCMX_ELIMIT, "gemv_pro: K=%lld above %d", (long long)K, GEMV_PRO_MAXK);
        SCMX_REQUIRE((reinterpret_cast<uintptr_t>(xbf) & 15) == 0 && (reinterpret_cast<uintptr_t>(nw) & 15) == 0, SCMX_EINVAL,
                     "gemv_pro: x and nw must be 16-byte aligned");
        xq = reinterpret_cast<const int8_t*>(xbf);          // stands in for the checks below; never read
        static const float one = 1.0f;
        if (xscale == nullptr) xscale = &one;                 // likewise
    }
    SCMX_REQUIRE(K > 0 && K % 128 == 0 && K <= (1 << 20), SCMX_EINVAL, "gemv: K=%lld must be a multiple of 128", (long long)K);
    SCMX_REQUIRE(N > 0 && N % 4 == 0 && N < (1ll << 30), SCMX_EINVAL, "gemv: N=%lld must be a multiple of 4", (long long)N);
    SCMX_REQUIRE(epi >= 0 && epi <= 3, SCMX_EINVAL, "gemv: epi=%d outside 0..3", epi);
    SCMX_REQUIRE(epi != 2 || res != nullptr, SCMX_EINVAL, "gemv: epi 2 needs res");
    SCMX_REQUIRE(epi == 0 || xscale != nullptr, SCMX_EINVAL, "gemv: xscale is NULL");
    SCMX_REQUIRE(K % (a.f.block * a.f.blocks_per_byte) == 0, SCMX_EINVAL,
                 "gemv: K=%lld not a multiple of block*codes_per_byte=%d", (long long)K, a.f.block * a.f.blocks_per_byte);
    SCMX_REQUIRE(a.f.block % 32 == 0 || 32 % a.f.block == 0, SCMX_EFORMAT, "gemv: block=%d must divide or be a multiple of 32",
                 a.f.block);
    SCMX_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 15) == 0 && (reinterpret_cast<uintptr_t>(xq) & 15) == 0, SCMX_EINVAL,
                 "gemv: codes and xq must be 16-byte aligned");
    int slots = 1;
    if (eidx) {
        SCMX_REQUIRE(n_routed >= 0 && n_routed + (shared >= 0 ? 1 : 0) >= 1, SCMX_EINVAL, "gemv: no slots");
        slots = n_routed + (shared >= 0 ? 1 : 0);
    }
    SCMX_REQUIRE(xstride == 0 || xstride == 1, SCMX_EINVAL, "gemv: xstride must be 0 or 1");
    a.xq = xq; a.xscale = xscale; a.codes = codes; a.bcodes = bcodes; a.wscale = wscale; a.res = res; a.eidx = eidx;
    a.out = out; a.N = (int)N; a.K = (int)K; a.epi = epi; a.n_routed = n_routed; a.shared = shared; a.xstride = xstride;
    a.bc_row_bytes = (int)(K / (a.f.block * a.f.blocks_per_byte));
    // ---- streaming kernel for dense GEMVs whose tiles satisfy the bulk-copy alignment rules
    // (matrices under 16 MB finish within a few microseconds either way and start faster with the register kernel below)
    if (!eidx && xbf == nullptr && (g_gemv_stream == 2 || g_gemv_stream == 3 || N * K / 2 >= (16ll << 20)) && K <= SG_X_BYTES && K % 32 == 0 && (a.bc_row_bytes % 4) == 0 && (reinterpret_cast<uintptr_t>(bcodes) & 15) == 0 &&
        g_gemv_stream) {
        int tr = 64;
        while (tr > 4 && ((int64_t)tr * (K / 2) > SG_STAGE_BYTES || (N + tr - 1) / tr < 96)) tr >>= 1;
        if ((int64_t)tr * (K / 2) <= SG_STAGE_BYTES && (int64_t)tr * a.bc_row_bytes <= SG_BC_BYTES && (K / (SG_NW / (tr / 4))) % 32 == 0) {
            StreamArgs sa;
            sa.g = a;
            sa.tr = tr;
            sa.n_tiles = (int)((N + tr - 1) / tr);
            sa.status = nullptr;
            sa.mode = g_gemv_stream == 2 ? 1 : 0;
            static int n_sm = 0;
            if (!n_sm) {
                int dev = 0;
                cudaGetDevice(&dev);
                cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
            }
            const int grid = sa.n_tiles < n_sm ? sa.n_tiles : n_sm;
            const size_t smem = SG_STAGES * (SG_STAGE_BYTES + SG_BC_BYTES) + SG_X_BYTES + 1280 + 8 * 2 * SG_STAGES + 16 + 128;
            const bool b32s = a.f.block % 32 == 0;
            static bool configured = false;
            if (!configured) {
                SCMX_CUDA_OK(cudaFuncSetAttribute(gemv_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                SCMX_CUDA_OK(cudaFuncSetAttribute(gemv_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured = true;
            }
            const int keep = g_use_pdl;
            g_use_pdl = pdl ? keep : 0;
            cudaError_t e = b32s ? launch_pdl(gemv_stream_kernel<true>, dim3(grid), dim3(SG_THREADS), smem, (cudaStream_t)stream, sa)
                                 : launch_pdl(gemv_stream_kernel<false>, dim3(grid), dim3(SG_THREADS), smem, (cudaStream_t)stream, sa);
            g_use_pdl = keep;
            if (e != cudaSuccess) {
                set_error("gemv_stream launch failed: %s", cudaGetErrorString(e));
                return SCMX_ECUDA;
            }
            return SCMX_OK;
        }
    }
    const int ksteps = (int)((K + 1023) / 1024);
    // A warp streams `steps` K-steps of 1024 codes for its 4 rows; the remaining K-steps are split over `sk` warps of
    // the CTA.  Prefer more loads in flight per warp (larger steps) only while the grid still has >= 16 warps per SM.
    const int64_t groups64 = N / 4;
    int steps = 1, sk = ksteps;
    for (int cand = 4; cand >= 1; cand >>= 1) {
        const int csk = (ksteps + cand - 1) / cand;
        if (csk <= 8 && (cand == 1 || groups64 * csk >= 148 * 16)) { steps = cand; sk = csk; break; }
    }
    while (sk > 8 && steps < 4) { steps *= 2; sk = (ksteps + steps - 1) / steps; }
    SCMX_REQUIRE(sk <= 8, SCMX_ELIMIT, "gemv: K=%lld too large (max 32768)", (long long)K);
    a.sk = sk;
    a.rg = 8 / sk < 1 ? 1 : 8 / sk;
    const int groups = (int)(N / 4);
    if (a.rg > groups) a.rg = groups;
    dim3 grid((groups + a.rg - 1) / a.rg, slots);
    const int threads = 32 * a.rg * a.sk;
    const bool b32 = a.f.block % 32 == 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (steps == 1) e = b32 ? launch_gemv<1, true>(a, grid, threads, pdl, st) : launch_gemv<1, false>(a, grid, threads, pdl, st);
    else if (steps == 2) e = b32 ? launch_gemv<2, true>(a, grid, threads, pdl, st) : launch_gemv<2, false>(a, grid, threads, pdl, st);
    else e = b32 ? launch_gemv<4, true>(a, grid, threads, pdl, st) : launch_gemv<4, false>(a, grid, threads, pdl, st);
    if (e != cudaSuccess) {
        set_error("gemv launch failed: %s", cudaGetErrorString(e));
        return SCMX_ECUDA;
    }
    return SCMX_OK;
}

extern "C" int scmx_gemv(const int8_t* xq, const float* xscale, const uint32_t* codes, const uint8_t* bcodes,
                         const float* wscale, int64_t N, int64_t K, const scmx_format* fmt, int epi, const uint16_t* res,
                         const int32_t* eidx, int n_routed, int shared, int xstride, void* out, int pdl, void* stream) {
    SCMX_REQUIRE(xq != nullptr, SCMX_EINVAL, "gemv: xq is NULL");
    return gemv_impl(xq, xscale, nullptr, nullptr, 0.0f, codes, bcodes, wscale, N, K, fmt, epi, res, eidx, n_routed, shared, xstride,
                     out, pdl, stream);
}

extern "C" int scmx_gemv_pro(const uint16_t* x, int pro, const uint16_t* nw, float eps, const uint32_t* codes,
                             const uint8_t* bcodes, const float* wscale, int64_t N, int64_t K, const scmx_format* fmt, int epi,
                             const uint16_t* res, const int32_t* eidx, int n_routed, int shared, int xstride, void* out, int pdl,
                             void* stream) {
    SCMX_REQUIRE(x != nullptr && (pro == 1 || (pro == 2 && nw != nullptr)), SCMX_EINVAL, "gemv_pro: pro=%d (1, or 2 with nw)", pro);
    SCMX_REQUIRE(epi != 0, SCMX_EINVAL, "gemv_pro: epi 0 has no scale to report; use the row kernel and scmx_gemv");
    return gemv_impl(nullptr, nullptr, x, pro == 2 ? nw : nullptr, eps, codes, bcodes, wscale, N, K, fmt, epi, res, eidx, n_routed,
                     shared, xstride, out, pdl, stream);
}
