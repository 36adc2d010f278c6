// One decode step of a dense (Qwen3-style) stack as ONE persistent kernel: every SM keeps a CTA resident for the whole
// step and the CTAs move through the phases of each layer together, separated by grid-wide barriers instead of kernel
// boundaries.  A batch-1 step is a chain of ~10 tiny dependent kernels per layer; launched separately (even from a CUDA
// graph, with programmatic dependent launch) each link costs a grid drain and a launch, about 5 us, while the weights it
// reads would take 1 us at HBM speed.  Here a link costs one barrier and the activations are re-quantized redundantly by every
// CTA in shared memory (instead of by a one-CTA kernel that everything waits for).  The phases are out-of-line functions with
// short loops, one copy each: the kernel runs every phase once per layer, so straight-line unrolled code would be fetched
// again from memory for every layer.
//
// Per layer (5 barriers):
//   P1  RMSNorm + INT8 of h (each CTA, shared memory; the first weight loads of every warp are already in flight) ->
//       q|k|v GEMV rows spread over all warps -> y (bf16)
//   P3  per (kv head, split) CTA: q/k RMSNorm + rotary embedding of the new token, cache append, attention over its
//       positions -> partial softmax states; the last split of a kv head to finish combines them -> o
//   P4  INT8 of o -> o-projection GEMV + residual -> h
//   P5  RMSNorm + INT8 of h -> gate|up GEMV with SwiGLU -> act
//   P6  INT8 of act -> down GEMV + residual -> h
// Arithmetic: the device functions of the stand-alone kernels (row kernels, GEMV, q/k/v epilogue, decode attention), so the
// step produces the same bits as the chain of those kernels.  Callers: e2e/decode.py:29-110 of the reference is the chain.
//
// Every wait is bounded (MK_WAIT_NS): a CTA that gives up raises the abort word, writes the status word and returns; the
// others see the abort word in their own waits and return too.  The launch is cooperative, so all CTAs are co-resident.
#include "scmx_attn_core.cuh"
#include "scmx_common.cuh"
#include "scmx_gemv_core.cuh"
#include "scmx_ptx.cuh"

namespace scmx {

constexpr int MK_THREADS = 256;
constexpr int MK_WARPS = MK_THREADS / 32;
constexpr int MK_MAXSTEPS = 6;                       // K <= 6144: a lane holds 32 codes of 4 rows per step
constexpr int MK_MAXK = 1024 * MK_MAXSTEPS;
constexpr int MK_MAXHQ = 32;
constexpr uint64_t MK_WAIT_NS = 500000000ull;        // 0.5 s

struct MkArgs {
    const scmx_decode_layer* layers;
    int n_layers, D, F, hq, hk, nsplit;
    float eps, scale;
    const float* inv_freq;
    const float* rope_cs;
    int64_t rope_rows, cap;
    const int32_t* pos_dev;
    uint16_t* h;          // bf16 [D] residual stream, in and out
    uint16_t* y;          // bf16 [(hq + 2 hk) d]
    uint16_t* act;        // bf16 [F]
    float* part;          // f32 [hq, nsplit, d + 2]
    uint16_t* o;          // bf16 [hq d] attention output
    int32_t* counters;    // int32 [hk], zero at launch and left zero: arrivals of the splits of a kv head
    uint32_t* bar;        // [0] arrivals, [1] abort word; both zero at launch
    int32_t* status;
    unsigned long long* trace;   // diagnostic: null, or CTA 0 stores its cycle counter at every phase boundary
    int n_trace;
    int trace_barrier;           // diagnostic: every CTA stores its arrival time at this barrier (1-based) after the marks
};

struct MkSmem {
    __align__(16) int8_t xq[MK_MAXK];
    __align__(16) uint4 xn[MK_MAXK / 8];
    float red[33];
    double dred[33];
    int ok;
};

__shared__ MkSmem sm;     // one instance per CTA, used by the out-of-line phase functions below

// ---- grid-wide barrier ------------------------------------------------------------------------------------------------------
__device__ __noinline__ bool grid_barrier(const MkArgs& a, uint32_t target) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(a.bar, 1u);
        int good = 1;
        uint64_t t0 = 0;
        for (uint32_t it = 0;; ++it) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.bar) : "memory");
            if (v >= target) break;
            if ((it & 255u) == 255u) {
                uint32_t ab;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(ab) : "l"(a.bar + 1) : "memory");
                if (ab) { good = 0; break; }
                const uint64_t now = globaltimer_ns();
                if (!t0) t0 = now;
                else if (now - t0 > MK_WAIT_NS) {
                    atomicExch(a.bar + 1, 1u);
                    atomicCAS((int*)a.status, 0, 100 + (int)(target / gridDim.x));   // which barrier gave up
                    good = 0;
                    break;
                }
            }
        }
        sm.ok = good;
    }
    __syncthreads();
    return sm.ok != 0;
}

__device__ __forceinline__ void mk_mark(const MkArgs& a, int& ti) {
    if (a.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && ti < a.n_trace) a.trace[ti] = (unsigned long long)clock64();
    ++ti;
}
// ---- activation prologues: bf16 row -> INT8 row in shared memory, returns the scale ------------------------------------------
__device__ __forceinline__ uint4 ldcg4(const uint4* p) { return __ldcg(p); }

// INT8 of the bf16 row staged in sm.xn (nv vectors of 8), arithmetic of act_quant; amax is this thread's partial maximum.
__device__ __forceinline__ float quantize_staged(int nv, float amax) {
    amax = block_max(amax, sm.red);
    float s, qi;
    quant_scale(amax, s, qi);
    for (int v = threadIdx.x; v < nv; v += MK_THREADS) {
        const uint4 r = sm.xn[v];
        const uint32_t x[4] = {r.x, r.y, r.z, r.w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[2 * j] = __uint_as_float(x[j] << 16);
            f[2 * j + 1] = __uint_as_float(x[j] & 0xFFFF0000u);
        }
        reinterpret_cast<uint2*>(sm.xq)[v] = make_uint2(quant4(f[0], f[1], f[2], f[3], qi), quant4(f[4], f[5], f[6], f[7], qi));
    }
    __syncthreads();
    return s;
}

__device__ __forceinline__ float amax8(const uint4& r) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) m = fmaxf(m, fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xFFFF0000u))));
    return m;
}

__device__ __forceinline__ float pro_act(const uint16_t* x, int K) {
    const int nv = K / 8;
    float amax = 0.0f;
    for (int v = threadIdx.x; v < nv; v += MK_THREADS) {
        const uint4 r = ldcg4(reinterpret_cast<const uint4*>(x) + v);
        sm.xn[v] = r;
        amax = fmaxf(amax, amax8(r));
    }
    return quantize_staged(nv, amax);
}

__device__ __forceinline__ float pro_norm(const uint16_t* x, const uint16_t* nw, float eps, int K) {
    const int nv = K / 8;
    double ss = 0.0;
    for (int v = threadIdx.x; v < nv; v += MK_THREADS) {
        const uint4 r = ldcg4(reinterpret_cast<const uint4*>(x) + v);
        sm.xn[v] = r;
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f0 = __uint_as_float(w[j] << 16), f1 = __uint_as_float(w[j] & 0xFFFF0000u);
            ss += sq_f64(f0) + sq_f64(f1);
        }
    }
    ss = block_sum(ss, sm.dred);
    const float inv = rms_inverse(ss, K, eps);
    float amax = 0.0f;
    const uint4* nw4 = reinterpret_cast<const uint4*>(nw);
    for (int v = threadIdx.x; v < nv; v += MK_THREADS) {       // the vectors this thread staged itself
        const uint4 r = sm.xn[v], wv = nw4[v];
        const uint32_t x4[4] = {r.x, r.y, r.z, r.w}, w[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t t = pack_bf16x2(__fmul_rn(bf16_lo(x4[j]), inv), __fmul_rn(bf16_hi(x4[j]), inv));
            o[j] = pack_bf16x2(__fmul_rn(bf16_lo(w[j]), bf16_lo(t)), __fmul_rn(bf16_hi(w[j]), bf16_hi(t)));
            amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(o[j])), fabsf(bf16_hi(o[j]))));
        }
        sm.xn[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    return quantize_staged(nv, amax);
}

// ---- GEMV: a warp computes 4 consecutive output rows over the whole K, in chunks of MK_UNROLL steps of 1024 codes -----------
// The chunks of a warp (row group after row group) form one sequence that is software-pipelined: the loads of chunk i + 1
// are issued before chunk i is expanded and accumulated, and nothing consumes a loaded value before all loads of its chunk
// are issued.  epi 1: out[n] = T(acc xs ws); 2: out[n] = T(res[n] + T(..)); 3: SwiGLU of rows [g0 g1 u0 u1].
constexpr int MK_UNROLL = 3;

struct RowChunk {
    uint4 w[MK_UNROLL][4];
    uint32_t bc[MK_UNROLL];       // lane l: block-code byte (l >> 2) of the step, of row (l & 3)
};

__device__ __forceinline__ void load_chunk(RowChunk& c, const uint32_t* __restrict__ codes, const uint8_t* __restrict__ bcodes,
                                           int n0, int s0, int steps, int wpr, int bcr, int lane) {
#pragma unroll
    for (int u = 0; u < MK_UNROLL; ++u) {
        if (s0 + u < steps) {
            const int k0 = ((s0 + u) * 32 + lane) * 32;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                c.w[u][q] = ldg_stream(reinterpret_cast<const uint4*>(codes + (size_t)(n0 + q) * wpr + k0 / 8));
            // the 32 lanes x 32 codes of a step span 8 block-code bytes per row: lane l fetches byte l >> 2 of row l & 3
            c.bc[u] = __ldg(bcodes + (size_t)(n0 + (lane & 3)) * bcr + (s0 + u) * 8 + (lane >> 2));
        }
    }
}

__device__ __forceinline__ void compute_chunk(const RowChunk& c, const int8_t* xq, int s0, int steps, int lane, int (&tot)[4]) {
    const uint32_t mlo = 0x03020100u, mhi = 0x0C080604u;      // 2 x E2M1 magnitudes 0 1 2 3 | 4 6 8 12
#pragma unroll
    for (int u = 0; u < MK_UNROLL; ++u) {
        if (s0 + u < steps) {
            const int k0 = ((s0 + u) * 32 + lane) * 32;
            const uint4 xa = *reinterpret_cast<const uint4*>(xq + k0);
            const uint4 xb = *reinterpret_cast<const uint4*>(xq + k0 + 16);
            const uint32_t x[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            const int sh = ((k0 >> 5) & 3) * 2;               // the lane's 32-block inside its block-code byte
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t ww[4] = {c.w[u][q].x, c.w[u][q].y, c.w[u][q].z, c.w[u][q].w};
                const uint32_t code = (__shfl_sync(0xffffffffu, c.bc[u], (lane & ~3) | q) >> sh) & 3u;
                // magnitudes of the positive and of the negative codes by sign-replicating byte permutes (a selector nibble with
                // its top bit set yields the replicated top bit of the selected byte, 0 for a magnitude), two DP4A chains
                int bp = 0, bn = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t w = ww[j], wx = w ^ 0x88888888u;
                    bp = dp4a_ss(x[2 * j], prmt(mlo, mhi, w), bp);
                    bn = dp4a_ss(x[2 * j], prmt(mlo, mhi, wx), bn);
                    bp = dp4a_ss(x[2 * j + 1], prmt(mlo, mhi, w >> 16), bp);
                    bn = dp4a_ss(x[2 * j + 1], prmt(mlo, mhi, wx >> 16), bn);
                }
                tot[q] += (bp - bn) << code;
            }
        }
    }
}

// One GEMV phase: the warp's first chunk of weights is requested, then the CTA computes the INT8 input row in shared memory
// (NORM: RMSNorm with weights nw first), then the chunks are consumed.  The weights do not depend on the activations, so
// their first round trip to memory runs under the prologue.
template <bool NORM>
__device__ __noinline__ void run_phase(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ bcodes,
                                       const float* __restrict__ wscale, int N, int K, const uint16_t* x, const uint16_t* nw,
                                       float eps, int epi, const uint16_t* res, uint16_t* out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // row groups are dealt warp-major, so that a job with fewer groups than warps still uses every SM
    const int gw = warp * gridDim.x + blockIdx.x, nw_ = gridDim.x * MK_WARPS;
    const int steps = K / 1024, wpr = K / 8, bcr = K / 128, groups = N / 4;
    const int8_t* xq = sm.xq;
    const bool work = gw < groups;
    RowChunk cur, nxt;
    int grp = gw, s0 = 0;
    if (work) load_chunk(cur, codes, bcodes, grp * 4, 0, steps, wpr, bcr, lane);
    const float xs = NORM ? pro_norm(x, nw, eps, K) : pro_act(x, K);     // every thread: contains CTA barriers
    if (!work) return;
    int tot[4] = {0, 0, 0, 0};
    for (;;) {
        // the chunk after this one: the next steps of the same rows, or the first steps of the warp's next row group
        int ngrp = grp, ns0 = s0 + MK_UNROLL;
        if (ns0 >= steps) {
            ngrp = grp + nw_;
            ns0 = 0;
        }
        const bool more = ngrp < groups;
        if (more) load_chunk(nxt, codes, bcodes, ngrp * 4, ns0, steps, wpr, bcr, lane);
        compute_chunk(cur, xq, s0, steps, lane, tot);
        if (ngrp != grp) {                                    // last chunk of the row group: reduce and write
            const int n0 = grp * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) tot[q] = warp_sum(tot[q]);
            // every lane holds the four totals; lane r finishes row r (selects, not indexing: the totals stay in registers)
            const int t_lo = (lane & 1) ? tot[1] : tot[0], t_hi = (lane & 1) ? tot[3] : tot[2];
            if (epi == 3) {
                if (lane < 2) {
                    const float gg = scale_acc(t_lo, xs, __ldg(wscale + n0 + lane));
                    const float uu = scale_acc(t_hi, xs, __ldg(wscale + n0 + lane + 2));
                    out[n0 / 2 + lane] = f32_to_bf16(swiglu_bf16(gg, uu));
                }
            } else if (lane < 4) {
                float y = scale_acc(lane < 2 ? t_lo : t_hi, xs, __ldg(wscale + n0 + lane));
                if (epi == 2) y = __fadd_rn(bf16_to_f32(__ldcg(res + n0 + lane)), y);
                out[n0 + lane] = f32_to_bf16(y);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) tot[q] = 0;
        }
        if (!more) break;
        cur = nxt;
        grp = ngrp;
        s0 = ns0;
    }
}

// ---- the new token's q (G heads), k, v of one key/value head: RMSNorm, rotary embedding (arithmetic of qkv_norm_kernel) ----
template <int G, int HD>
struct QkvSmem {
    float vals[(G + 2) * HD];
    float inv[G + 1];
    float cs[HD / 2], sn[HD / 2];
    __align__(16) uint16_t q[G * HD];
    __align__(16) uint16_t k[HD];
    __align__(16) uint16_t v[HD];
};

template <int G, int HD>
__device__ __forceinline__ void qkv_prepare(QkvSmem<G, HD>& qs, const MkArgs& a, const scmx_decode_layer& L, int kvh, int64_t pos) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int half = HD / 2, NE = (G + 2) * HD;
    for (int e = tid; e < NE; e += MK_THREADS) {
        const int hh = e / HD, dd = e - hh * HD;
        const int src = hh < G ? (kvh * G + hh) * HD : (hh == G ? (a.hq + kvh) * HD : (a.hq + a.hk + kvh) * HD);
        qs.vals[e] = bf16_to_f32(__ldcg(a.y + src + dd));
    }
    for (int i = tid; i < half; i += MK_THREADS) {
        if (a.rope_cs != nullptr && pos < a.rope_rows) {
            qs.cs[i] = a.rope_cs[pos * HD + i];
            qs.sn[i] = a.rope_cs[pos * HD + half + i];
        } else {
            const float ang = __fmul_rn((float)pos, a.inv_freq[i]);
            double s, c;
            sincos((double)ang, &s, &c);
            qs.cs[i] = (float)c;
            qs.sn[i] = (float)s;
        }
    }
    __syncthreads();
    for (int hh = warp; hh < G + 1; hh += MK_WARPS) {
        double ss = 0.0;
        for (int i = lane; i < HD; i += 32) {
            const double x = (double)qs.vals[hh * HD + i];
            ss += x * x;
        }
        ss = warp_sum(ss);
        if (lane == 0) qs.inv[hh] = rms_inverse(ss, HD, a.eps);
    }
    __syncthreads();
    auto normed = [&](int hh, int dd) -> float {
        const uint16_t* w = hh < G ? L.q_norm : L.k_norm;
        return rbf(__fmul_rn(bf16_to_f32(w[dd]), rbf(__fmul_rn(qs.vals[hh * HD + dd], qs.inv[hh]))));
    };
    for (int e = tid; e < NE; e += MK_THREADS) {
        const int hh = e / HD, dd = e - hh * HD;
        if (hh > G) {
            qs.v[dd] = f32_to_bf16(qs.vals[e]);
            continue;
        }
        const bool lo = dd < half;
        const float self = normed(hh, dd), other = normed(hh, lo ? dd + half : dd - half);
        const int i = lo ? dd : dd - half;
        const float r = lo ? rbf(__fsub_rn(__fmul_rn(self, qs.cs[i]), __fmul_rn(other, qs.sn[i])))
                           : rbf(__fadd_rn(__fmul_rn(other, qs.sn[i]), __fmul_rn(self, qs.cs[i])));
        if (hh < G) qs.q[hh * HD + dd] = f32_to_bf16(r);
        else qs.k[dd] = f32_to_bf16(r);
    }
    __syncthreads();
}

// ---- the kernel ------------------------------------------------------------------------------------------------------------
template <int G, int HD>
__global__ void __launch_bounds__(MK_THREADS, 1) decode_step_kernel(const MkArgs a) {
    __shared__ QkvSmem<G, HD> qs;
    __shared__ AttnSmem<G, HD> as;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int D = a.D, F = a.F, QD = a.hq * HD, NQKV = (a.hq + 2 * a.hk) * HD;
    uint32_t target = 0;

    int64_t pos = a.pos_dev[0];
    pos = pos < 0 ? 0 : pos;
    const bool in_cache = pos < a.cap;
    int64_t T = in_cache ? pos + 1 : a.cap;
    int64_t chunk;
    int active;
    attn_chunking(T, a.nsplit, chunk, active);
    constexpr int stride = HD + 2;

    int ti = 0;
#define MK_MARK()                                                                                   \
    do {                                                                                            \
        mk_mark(a, ti);                                                                             \
    } while (0)
#define MK_BARRIER()                                          \
    do {                                                      \
        MK_MARK();                                            \
        target += gridDim.x;                                  \
        if (a.trace != nullptr && tid == 0 && (int)(target / gridDim.x) == a.trace_barrier)                      \
            a.trace[a.n_trace + blockIdx.x] = globaltimer_ns();                                             \
        if (!grid_barrier(a, target)) return;         \
        MK_MARK();                                            \
    } while (0)

    for (int li = 0; li < a.n_layers; ++li) {
        const scmx_decode_layer L = a.layers[li];             // by value: the pointers sit in registers for the whole layer
        // P1: input RMSNorm + INT8, q|k|v projection
        if (li > 0) MK_BARRIER();                             // h of the previous layer complete
        run_phase<true>(L.codes[0], L.bcodes[0], L.wscale[0], NQKV, D, a.h, L.ln_in, a.eps, 1, nullptr, a.y);
        // P3: attention of one (kv head, split) per CTA
        MK_BARRIER();
        {
            const int kvh = blockIdx.x % a.hk, split = blockIdx.x / a.hk;
            if (split < active) {                             // uniform over the CTA
                qkv_prepare<G, HD>(qs, a, L, kvh, pos);
                MK_MARK();
                uint16_t* kc = L.k_cache + (size_t)kvh * a.cap * HD;
                uint16_t* vc = L.v_cache + (size_t)kvh * a.cap * HD;
                if (split == 0 && in_cache && tid < HD / 8) {
                    reinterpret_cast<uint4*>(kc + pos * HD)[tid] = reinterpret_cast<const uint4*>(qs.k)[tid];
                    reinterpret_cast<uint4*>(vc + pos * HD)[tid] = reinterpret_cast<const uint4*>(qs.v)[tid];
                }
                const int64_t t0 = (int64_t)split * chunk, t1 = t0 + chunk < T ? t0 + chunk : T;
                attn_split<G, HD>(qs.q, kc, vc, t0, t1, in_cache ? pos : -1, qs.k, qs.v, a.scale,
                                  a.part + ((size_t)kvh * G * a.nsplit + split) * stride, (size_t)a.nsplit * stride, as);
                MK_MARK();
                // the last split of this kv head to finish combines them (the arithmetic of attn_combine) into o
                __syncthreads();
                if (tid == 0) {                               // one fence orders the CTA's partials before the ticket
                    __threadfence();
                    sm.ok = atomicAdd(a.counters + kvh, 1);
                    __threadfence();
                }
                __syncthreads();
                if (sm.ok == active - 1) {
                    attn_combine_cta<G, HD>(a.part + (size_t)kvh * G * a.nsplit * stride, a.nsplit, active,
                                            a.o + (size_t)kvh * G * HD, as);
                    if (tid == 0) a.counters[kvh] = 0;
                }
            }
        }
        // P4: combine the splits, INT8 of o, o-projection + residual
        MK_BARRIER();
        run_phase<false>(L.codes[1], L.bcodes[1], L.wscale[1], D, QD, a.o, nullptr, 0.0f, 2, a.h, a.h);
        // P5: post-attention RMSNorm + INT8, gate|up projection with SwiGLU
        MK_BARRIER();
        run_phase<true>(L.codes[2], L.bcodes[2], L.wscale[2], 2 * F, D, a.h, L.ln_post, a.eps, 3, nullptr, a.act);
        // P6: INT8 of act, down projection + residual
        MK_BARRIER();
        run_phase<false>(L.codes[3], L.bcodes[3], L.wscale[3], D, F, a.act, nullptr, 0.0f, 2, a.h, a.h);
    }
#undef MK_BARRIER
#undef MK_MARK
}

}  // namespace scmx

using namespace scmx;

static unsigned long long* g_trace = nullptr;
static int g_n_trace = 0;
extern "C" int scmx_set_decode_trace(unsigned long long* device_buf, int n) {
    g_trace = n > 0 ? device_buf : nullptr;
    g_n_trace = g_trace ? n : 0;
    return SCMX_OK;
}

extern "C" int scmx_decode_step_dense(const scmx_decode_layer* layers, int n_layers, int D, int F, int hq, int hk, int d, float eps,
                                      float scale, const float* inv_freq, const float* rope_table, int64_t rope_rows,
                                      int64_t capacity, const int32_t* pos_dev, uint16_t* h, uint16_t* y, uint16_t* act,
                                      uint16_t* o, float* partials, int nsplit, int32_t* counters, uint32_t* barrier,
                                      int32_t* status, void* stream) {
    SCMX_REQUIRE(layers && pos_dev && h && y && act && o && partials && counters && barrier && status && inv_freq, SCMX_EINVAL, "decode_step: null buffer");
    SCMX_REQUIRE(n_layers > 0 && hq > 0 && hk > 0 && hq % hk == 0 && hq <= MK_MAXHQ, SCMX_EINVAL, "decode_step: hq=%d hk=%d", hq, hk);
    SCMX_REQUIRE(d == 128, SCMX_ELIMIT, "decode_step: head size %d (128)", d);
    const int G = hq / hk;
    SCMX_REQUIRE(G == 1 || G == 2 || G == 4, SCMX_ELIMIT, "decode_step: %d query heads per key/value head (1, 2 or 4)", G);
    SCMX_REQUIRE(D % 1024 == 0 && F % 1024 == 0 && (hq * d) % 1024 == 0 && D <= MK_MAXK && F <= MK_MAXK && hq * d <= MK_MAXK,
                 SCMX_ELIMIT, "decode_step: widths D=%d F=%d hq*d=%d must be multiples of 1024 up to %d", D, F, hq * d, MK_MAXK);
    SCMX_REQUIRE(capacity >= 1 && nsplit >= 1 && nsplit <= 32, SCMX_EINVAL, "decode_step: capacity=%lld nsplit=%d", (long long)capacity, nsplit);
    static int coop_dev[64] = {};            // 0 unknown, 1 supported, -1 not: per device
    const int dev = current_device();
    SCMX_REQUIRE(dev >= 0, SCMX_ECUDA, "decode_step: no current CUDA device (ordinal 0..63)");
    if (!coop_dev[dev]) {
        int c = 0;
        SCMX_CUDA_OK(cudaDeviceGetAttribute(&c, cudaDevAttrCooperativeLaunch, dev));
        coop_dev[dev] = c ? 1 : -1;
    }
    const int coop = coop_dev[dev] > 0, n_sm = sm_count();
    SCMX_REQUIRE(coop, SCMX_EDEVICE, "decode_step: the device does not support cooperative launches");
    SCMX_REQUIRE(hk * nsplit <= n_sm, SCMX_EINVAL, "decode_step: hk * nsplit = %d exceeds the %d CTAs of the grid", hk * nsplit, n_sm);
    MkArgs a;
    a.layers = layers; a.n_layers = n_layers; a.D = D; a.F = F; a.hq = hq; a.hk = hk; a.nsplit = nsplit; a.eps = eps; a.scale = scale;
    a.inv_freq = inv_freq; a.rope_cs = rope_table; a.rope_rows = rope_table ? rope_rows : 0; a.cap = capacity; a.pos_dev = pos_dev;
    a.h = h; a.y = y; a.act = act; a.o = o; a.counters = counters; a.part = partials; a.bar = barrier; a.status = status;
    a.trace = g_trace; a.n_trace = g_n_trace & 0xFFFF; a.trace_barrier = g_n_trace >> 16;
    cudaStream_t st = (cudaStream_t)stream;
    SCMX_CUDA_OK(cudaMemsetAsync(barrier, 0, 2 * sizeof(uint32_t), st));
    // tickets taken by a step that gave up on a barrier are not returned: start every step from zero
    SCMX_CUDA_OK(cudaMemsetAsync(counters, 0, (size_t)hk * sizeof(int32_t), st));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)n_sm);
    cfg.blockDim = dim3(MK_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = G == 1 ? cudaLaunchKernelEx(&cfg, decode_step_kernel<1, 128>, a)
                  : G == 2 ? cudaLaunchKernelEx(&cfg, decode_step_kernel<2, 128>, a)
                           : cudaLaunchKernelEx(&cfg, decode_step_kernel<4, 128>, a);
    SCMX_PDL_OK("decode_step_kernel", e);
    return SCMX_OK;
}
