// Device functions of the batch-1 decode attention, shared by the stand-alone kernel and the persistent decode kernel so
// that both produce the same bits: position chunking, one (key/value head, split) task with a float32 online softmax,
// and the combination of the splits.
#pragma once
#include "scmx_common.cuh"

namespace scmx {

constexpr int AD_THREADS = 256;        // 8 warps x 4 position slots x 8 lanes per position
constexpr int AD_WARPS = AD_THREADS / 32;
constexpr int AD_GROUP = AD_WARPS * 4;  // positions the CTA consumes together
constexpr int AD_MIN_CHUNK = 32;       // positions per split at least: short sequences use the first few splits only
constexpr int AD_UNROLL = 2;           // groups of positions whose loads are in flight together
constexpr float LOG2E = 1.4426950408889634f;

template <int G, int D>
struct AttnSmem {
    float acc[AD_WARPS][G][D];
    float ml[AD_WARPS][G][2];
    float cml[G * 32][2];     // combination: running maximum and sum of every (head, split)
    float coef[G][33];        // weight of every split, [32] = the normalizer
};

// T positions over nsplit splits -> positions per split (a multiple of 16) and the number of splits that have work.
__device__ __forceinline__ void attn_chunking(int64_t T, int nsplit, int64_t& chunk, int& active) {
    chunk = (T + nsplit - 1) / nsplit;
    chunk = chunk < AD_MIN_CHUNK ? AD_MIN_CHUNK : ((chunk + 15) & ~(int64_t)15);
    active = (int)((T + chunk - 1) / chunk);
}

// merge (m2, l2, a2) into (m, l, a): two partial softmax states over disjoint positions
template <int E>
__device__ __forceinline__ void merge_state(float& m, float& l, float (&a)[E], float m2, float l2, const float (&a2)[E]) {
    const float mn = fmaxf(m, m2);
    if (mn == -INFINITY) return;
    const float c1 = exp2f(m - mn), c2 = exp2f(m2 - mn);
    l = l * c1 + l2 * c2;
#pragma unroll
    for (int i = 0; i < E; ++i) a[i] = a[i] * c1 + a2[i] * c2;
    m = mn;
}

// One (key/value head, split) task, run by the first AD_THREADS threads of the CTA (every thread of the CTA must call it:
// it contains __syncthreads).  q: bf16 [G][D] of the G query heads sharing this key/value head; kb / vb: the head's cache
// rows [cap][D]; positions [t0, t1).  Position t_new (or -1) is read from knew / vnew (bf16 [D]) instead of the cache.
// q, knew, vnew may point to shared or global memory.  Writes the G partial states to part + g * part_stride_g:
// D unnormalized outputs, the running maximum (log2 domain), the running sum.
template <int G, int D>
__device__ __forceinline__ void attn_split(const uint16_t* q, const uint16_t* kb, const uint16_t* vb, int64_t t0, int64_t t1,
                                           int64_t t_new, const uint16_t* knew, const uint16_t* vnew, float scale, float* part,
                                           size_t part_stride_g, AttnSmem<G, D>& sm) {
    constexpr int E = D / 8;                  // elements per lane
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, slot = lane >> 3, l8 = lane & 7;
    if (tid < AD_THREADS) {
        float qf[G][E], acc[G][E], m[G], l[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const uint16_t* qp = q + (size_t)g * D + l8 * E;
#pragma unroll
            for (int i = 0; i < E; ++i) {
                qf[g][i] = bf16_to_f32(qp[i]) * (scale * LOG2E);
                acc[g][i] = 0.0f;
            }
            m[g] = -INFINITY;
            l[g] = 0.0f;
        }
        // the trip count is uniform over the warp (the shuffles below need every lane); slots past the end are masked.
        // AD_UNROLL groups of AD_GROUP positions per trip: the loads of all groups are issued before the first one is consumed,
        // so that a CTA keeps AD_UNROLL x AD_GROUP x 2 rows in flight; the positions of a thread are consumed in ascending order.
        for (int64_t tb = t0 + warp * 4; tb < t1; tb += AD_GROUP * AD_UNROLL) {
            uint4 kw[AD_UNROLL][E / 8], vw[AD_UNROLL][E / 8];
#pragma unroll
            for (int u = 0; u < AD_UNROLL; ++u) {
                const int64_t t = tb + AD_GROUP * u + slot;
                const uint16_t* kp = (t == t_new) ? knew + l8 * E : kb + t * D + l8 * E;
                const uint16_t* vp = (t == t_new) ? vnew + l8 * E : vb + t * D + l8 * E;
#pragma unroll
                for (int c = 0; c < E / 8; ++c) {
                    kw[u][c] = make_uint4(0, 0, 0, 0);
                    vw[u][c] = make_uint4(0, 0, 0, 0);
                    if (t < t1) {
                        kw[u][c] = *reinterpret_cast<const uint4*>(kp + 8 * c);
                        vw[u][c] = *reinterpret_cast<const uint4*>(vp + 8 * c);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < AD_UNROLL; ++u) {
                if (tb + AD_GROUP * u < t1) {         // uniform over the warp
                    const bool valid = tb + AD_GROUP * u + slot < t1;
                    float kf[E], vf[E];
#pragma unroll
                    for (int c = 0; c < E / 8; ++c) {
                        const uint32_t ku[4] = {kw[u][c].x, kw[u][c].y, kw[u][c].z, kw[u][c].w};
                        const uint32_t vu[4] = {vw[u][c].x, vw[u][c].y, vw[u][c].z, vw[u][c].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            kf[8 * c + 2 * i] = __uint_as_float(ku[i] << 16);
                            kf[8 * c + 2 * i + 1] = __uint_as_float(ku[i] & 0xFFFF0000u);
                            vf[8 * c + 2 * i] = __uint_as_float(vu[i] << 16);
                            vf[8 * c + 2 * i + 1] = __uint_as_float(vu[i] & 0xFFFF0000u);
                        }
                    }
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        float s = 0.0f;
#pragma unroll
                        for (int i = 0; i < E; ++i) s = fmaf(qf[g][i], kf[i], s);
                        s += __shfl_xor_sync(0xffffffffu, s, 1);
                        s += __shfl_xor_sync(0xffffffffu, s, 2);
                        s += __shfl_xor_sync(0xffffffffu, s, 4);
                        if (valid) {
                            const float mn = fmaxf(m[g], s);
                            const float corr = exp2f(m[g] - mn), p = exp2f(s - mn);
                            l[g] = l[g] * corr + p;
#pragma unroll
                            for (int i = 0; i < E; ++i) acc[g][i] = acc[g][i] * corr + p * vf[i];
                            m[g] = mn;
                        }
                    }
                }
            }
        }
        // merge the 4 position slots of a warp
#pragma unroll
        for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float m2 = __shfl_xor_sync(0xffffffffu, m[g], off), l2 = __shfl_xor_sync(0xffffffffu, l[g], off);
                float a2[E];
#pragma unroll
                for (int i = 0; i < E; ++i) a2[i] = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
                merge_state<E>(m[g], l[g], acc[g], m2, l2, a2);
            }
        }
        if (slot == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
#pragma unroll
                for (int i = 0; i < E; ++i) sm.acc[warp][g][l8 * E + i] = acc[g][i];
                if (l8 == 0) {
                    sm.ml[warp][g][0] = m[g];
                    sm.ml[warp][g][1] = l[g];
                }
            }
        }
    }
    __syncthreads();
    // merge the warps; thread e < D owns output element e of every q head of this kv head
    if (tid < AD_THREADS) {
        for (int g = 0; g < G; ++g) {
            float mm = -INFINITY;
            for (int w = 0; w < AD_WARPS; ++w) mm = fmaxf(mm, sm.ml[w][g][0]);
            float ll = 0.0f, av = 0.0f;
            for (int w = 0; w < AD_WARPS; ++w) {
                const float c = mm == -INFINITY ? 0.0f : exp2f(sm.ml[w][g][0] - mm);
                ll += sm.ml[w][g][1] * c;
                if (tid < D) av += sm.acc[w][g][tid] * c;
            }
            float* p = part + (size_t)g * part_stride_g;
            if (tid < D) p[tid] = av;
            if (tid == 0) {
                p[D] = mm;
                p[D + 1] = ll;
            }
        }
    }
}

// The G heads of one key/value head from the partial states of their `active` splits, by the whole CTA (every thread must
// call it): out[g * D + e] = sum_s a_s[e] c_s / sum_s l_s c_s with c_s = 2^(m_s - max m), splits in ascending order.
// part: the partial states of head 0 of the group (head g at + g * nsplit * (D + 2) floats); active <= 32.
template <int G, int D>
__device__ __forceinline__ void attn_combine_cta(const float* part, int nsplit, int active, uint16_t* out, AttnSmem<G, D>& sm) {
    constexpr int stride = D + 2;
    const int tid = threadIdx.x, nt = blockDim.x;
    // the partial outputs of this thread's first element do not depend on the weights: request them before anything else, so
    // that their round trip overlaps the one of the running maxima / sums
    float v0[32];
    const bool first = tid < G * D;
    {
        const int g = tid / D, e = tid - g * D;
        const float* p = part + (size_t)g * nsplit * stride + e;
#pragma unroll
        for (int s = 0; s < 32; ++s) v0[s] = (first && s < active) ? __ldcg(p + s * stride) : 0.0f;
    }
    for (int i = tid; i < G * active; i += nt) {
        const int g = i / active, s = i - g * active;
        const float* p = part + ((size_t)g * nsplit + s) * stride;
        sm.cml[g * 32 + s][0] = __ldcg(p + D);
        sm.cml[g * 32 + s][1] = __ldcg(p + D + 1);
    }
    __syncthreads();
    for (int g = tid; g < G; g += nt) {
        float mm = -INFINITY;
        for (int s = 0; s < active; ++s) mm = fmaxf(mm, sm.cml[g * 32 + s][0]);
        float ll = 0.0f;
        for (int s = 0; s < active; ++s) {
            const float ms = sm.cml[g * 32 + s][0];
            const float c = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
            ll += sm.cml[g * 32 + s][1] * c;
            sm.coef[g][s] = c;
        }
        sm.coef[g][32] = ll;
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += nt) {
        const int g = i / D, e = i - g * D;
        float av = 0.0f;
        if (i == tid) {
#pragma unroll
            for (int s = 0; s < 32; ++s)
                if (s < active) av += v0[s] * sm.coef[g][s];
        } else {
            const float* p = part + (size_t)g * nsplit * stride + e;
            float v[32];
#pragma unroll
            for (int s = 0; s < 32; ++s) v[s] = s < active ? __ldcg(p + s * stride) : 0.0f;   // all loads in flight at once
#pragma unroll
            for (int s = 0; s < 32; ++s)
                if (s < active) av += v[s] * sm.coef[g][s];
        }
        out[i] = f32_to_bf16(av / sm.coef[g][32]);
    }
}

}  // namespace scmx
