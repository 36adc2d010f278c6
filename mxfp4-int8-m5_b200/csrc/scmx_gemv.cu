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

// scmx_gemv_multi.cu
int gemv_stream_single(const int8_t* xq, const float* xscale, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                       int64_t N, int64_t K, const DevFormat& f, int epi, const uint16_t* res, void* out, int pdl, cudaStream_t st);

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


// The 8 codes of word w against activations xa (codes 0..3) and xb (codes 4..7).  The byte permute's selector nibble is the code
// itself: with its top bit (the sign) set, the permute returns the replicated top bit of the selected byte, i.e. 0 for a
// magnitude; so prmt(LUT, w) holds the magnitudes of the positive codes and prmt(LUT, w ^ 0x88888888) those of the negative
// ones.  Two DP4A chains, subtracted by the caller: no negated copy of the activations, no sign-select permute.
__device__ __forceinline__ void word_pn(uint32_t w, uint32_t xa, uint32_t xb, uint32_t mlo, uint32_t mhi, int& ap, int& an) {
    const uint32_t wx = w ^ 0x88888888u;
    ap = dp4a_ss(xa, prmt(mlo, mhi, w), ap);
    an = dp4a_ss(xa, prmt(mlo, mhi, wx), an);
    ap = dp4a_ss(xb, prmt(mlo, mhi, w >> 16), ap);
    an = dp4a_ss(xb, prmt(mlo, mhi, wx >> 16), an);
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
            if (PRO == 2) ss += sq_f64(f0) + sq_f64(f1);
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
                const uint32_t t = pack_bf16x2(__fmul_rn(bf16_lo(x[j]), inv), __fmul_rn(bf16_hi(x[j]), inv));
                o[j] = pack_bf16x2(__fmul_rn(bf16_lo(w[j]), bf16_lo(t)), __fmul_rn(bf16_hi(w[j]), bf16_hi(t)));
                amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(o[j])), fabsf(bf16_hi(o[j]))));
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
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t ww[4] = {w[s][r].x, w[s][r].y, w[s][r].z, w[s][r].w};
            if (B32) {
                const int blk = block_of(a.f, k0s[s]);
                const uint32_t code = (bc[s][r] >> ((blk & a.f.pb_mask) << a.f.bc_shift)) & a.f.bc_mask;
                int bp = 0, bn = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) word_pn(ww[j], x[2 * j], x[2 * j + 1], a.f.mag_lo, a.f.mag_hi, bp, bn);
                tot[r] += a.f.pow2 ? ((bp - bn) << code) : (bp - bn) * (int)fmt_mult(a.f, code);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int bi = (8 * j) >> a.f.block_shift;   // block index inside the lane's 32 codes
                    const uint32_t code = (bc[s][r] >> (bi << a.f.bc_shift)) & a.f.bc_mask;
                    int bp = 0, bn = 0;
                    word_pn(ww[j], x[2 * j], x[2 * j + 1], a.f.mag_lo, a.f.mag_hi, bp, bn);
                    tot[r] += (bp - bn) * (int)fmt_mult(a.f, code);
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

static int g_gemv_stream = 1;      // 0 never, 1 for matrices of 16 MB and more, 2 whenever the shape allows
extern "C" int scmx_set_gemv_stream(int mode) {
    SCMX_REQUIRE(mode >= 0 && mode <= 2, SCMX_EINVAL, "set_gemv_stream: mode=%d (0 off, 1 automatic, 2 whenever the shape allows)", mode);
    g_gemv_stream = mode;
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
    // ---- streaming kernel (bulk-copy ring, persistent CTAs) for dense GEMVs that satisfy its alignment rules; matrices
    // under 16 MB finish within a few microseconds either way and start faster with the register kernel below
    if (!eidx && xbf == nullptr && g_gemv_stream && (g_gemv_stream == 2 || N * K / 2 >= (16ll << 20)) && K <= 8192 &&
        (a.bc_row_bytes % 4) == 0 && (a.f.block == 8 || a.f.block == 16 || a.f.block % 32 == 0) && a.f.block_shift >= 0 &&
        ((reinterpret_cast<uintptr_t>(bcodes) | reinterpret_cast<uintptr_t>(wscale)) & 15) == 0) {
        rc = gemv_stream_single(xq, xscale, codes, bcodes, wscale, N, K, a.f, epi, res, out, pdl, (cudaStream_t)stream);
        if (rc != SCMX_ELIMIT) return rc;         // SCMX_ELIMIT: the shape does not fit the streaming kernel
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
