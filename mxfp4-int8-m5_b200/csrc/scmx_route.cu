// MoE routing on the device: router softmax + top-k, and the counting sort of token-expert assignments by expert
// with segment offsets and M-tile starts (the inputs of the grouped GEMM's tile scheduler).
#include <cooperative_groups.h>
#include <float.h>
#include "scmx_common.cuh"

namespace scmx {

// One CTA sorts all R = M*topk assignments: shared-memory histogram, serial prefix over E <= 1024 experts, then a
// scatter where every assignment takes the next free row of its expert.  Row order inside an expert segment is
// arbitrary (atomics), which changes no result because every sorted row is computed independently.
__global__ void __launch_bounds__(1024) route_sort_kernel(const int32_t* __restrict__ inds, int R, int topk, int E, int tm,
                                                          int32_t* __restrict__ pos, int32_t* __restrict__ tok,
                                                          int32_t* __restrict__ esorted, int32_t* __restrict__ off,
                                                          int32_t* __restrict__ tstart) {
    __shared__ unsigned cnt[1024];
    __shared__ unsigned cur[1024];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, nt = blockDim.x;
    for (int e = tid; e < E; e += nt) cnt[e] = 0;
    __syncthreads();
    for (int i = tid; i < R; i += nt) {
        const unsigned e = (unsigned)inds[i];
        if (e < (unsigned)E) atomicAdd(&cnt[e], 1u);
    }
    __syncthreads();
    if (tid < 32) {
        // warp-level exclusive scan over experts in chunks of 32
        unsigned o = 0, t = 0;
        for (int base = 0; base < E; base += 32) {
            const int e = base + tid;
            const unsigned c = e < E ? cnt[e] : 0u;
            const unsigned ti = (c + tm - 1) / tm;
            unsigned so = c, st = ti;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const unsigned a = __shfl_up_sync(0xffffffffu, so, d), b = __shfl_up_sync(0xffffffffu, st, d);
                if (tid >= d) { so += a; st += b; }
            }
            if (e < E) {
                off[e] = (int)(o + so - c);
                tstart[e] = (int)(t + st - ti);
                cur[e] = o + so - c;
            }
            o += __shfl_sync(0xffffffffu, so, 31);
            t += __shfl_sync(0xffffffffu, st, 31);
        }
        if (tid == 0) { off[E] = (int)o; tstart[E] = (int)t; }
    }
    __syncthreads();
    for (int i = tid; i < R; i += nt) {
        const unsigned e = (unsigned)inds[i];
        if (e < (unsigned)E) {
            const unsigned p = atomicAdd(&cur[e], 1u);
            pos[i] = (int)p;
            tok[p] = i / topk;
            esorted[p] = (int)e;
        }
    }
    for (int p = R + tid; p < R + tm; p += nt) tok[p] = 0;   // padding rows gather token 0 and are never stored
}

// The same sort by a thread-block cluster of RS_CLUSTER CTAs for large R: every CTA histograms a contiguous chunk of the
// assignments in its own shared memory; after a cluster barrier each CTA reads the other histograms through distributed
// shared memory, computes the segment offsets (redundantly) and its own first free row per expert (the rows of lower-ranked
// CTAs come first), and scatters its chunk.  No global scratch; order inside a segment is still arbitrary.
constexpr int RS_CLUSTER = 8;

__global__ void __launch_bounds__(1024) route_sort_cluster_kernel(const int32_t* __restrict__ inds, int R, int topk, int E, int tm,
                                                                  int32_t* __restrict__ pos, int32_t* __restrict__ tok,
                                                                  int32_t* __restrict__ esorted, int32_t* __restrict__ off,
                                                                  int32_t* __restrict__ tstart) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ unsigned cnt[1024];      // this CTA's chunk
    __shared__ unsigned tot[1024];      // all chunks
    __shared__ unsigned cur[1024];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, nt = blockDim.x;
    const unsigned rank = cluster.block_rank(), nblk = cluster.num_blocks();
    const int per = (R + (int)nblk - 1) / (int)nblk;
    const int i0 = (int)rank * per, i1 = min(R, i0 + per);
    for (int e = tid; e < E; e += nt) cnt[e] = 0;
    __syncthreads();
    for (int i = i0 + tid; i < i1; i += nt) {
        const unsigned e = (unsigned)inds[i];
        if (e < (unsigned)E) atomicAdd(&cnt[e], 1u);
    }
    cluster.sync();
    for (int e = tid; e < E; e += nt) {
        unsigned all = 0, before = 0;
        for (unsigned r = 0; r < nblk; ++r) {
            const unsigned c = cluster.map_shared_rank(cnt, r)[e];
            all += c;
            if (r < rank) before += c;
        }
        tot[e] = all;
        cur[e] = before;                 // plus the segment offset, added below
    }
    cluster.sync();                      // no CTA leaves (or overwrites cnt) while another still reads its histogram
    if (tid < 32) {
        unsigned o = 0, t = 0;
        for (int base = 0; base < E; base += 32) {
            const int e = base + tid;
            const unsigned c = e < E ? tot[e] : 0u;
            const unsigned ti = (c + tm - 1) / tm;
            unsigned so = c, st = ti;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const unsigned a = __shfl_up_sync(0xffffffffu, so, d), b = __shfl_up_sync(0xffffffffu, st, d);
                if (tid >= d) { so += a; st += b; }
            }
            if (e < E) {
                if (rank == 0) {
                    off[e] = (int)(o + so - c);
                    tstart[e] = (int)(t + st - ti);
                }
                cur[e] += o + so - c;
            }
            o += __shfl_sync(0xffffffffu, so, 31);
            t += __shfl_sync(0xffffffffu, st, 31);
        }
        if (tid == 0 && rank == 0) { off[E] = (int)o; tstart[E] = (int)t; }
    }
    __syncthreads();
    for (int i = i0 + tid; i < i1; i += nt) {
        const unsigned e = (unsigned)inds[i];
        if (e < (unsigned)E) {
            const unsigned p = atomicAdd(&cur[e], 1u);
            pos[i] = (int)p;
            tok[p] = i / topk;
            esorted[p] = (int)e;
        }
    }
    if (rank == 0)
        for (int p = R + tid; p < R + tm; p += nt) tok[p] = 0;
}

// One warp per token: softmax over E <= 32 PER logits in float32, then topk rounds of warp arg-max (ties -> lower expert id).
template <int PER>
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, int64_t M, int E, int topk,
                                                          int32_t* __restrict__ inds, uint16_t* __restrict__ scores,
                                                          float* __restrict__ scores_f32) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= M) return;
    const float* lg = logits + t * E;
    float p[PER];
    float mx = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * 32 + lane;
        p[j] = e < E ? lg[e] : -FLT_MAX;
        mx = fmaxf(mx, p[j]);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * 32 + lane;
        p[j] = e < E ? expf(__fsub_rn(p[j], mx)) : 0.0f;
        sum += p[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * 32 + lane;
        p[j] = e < E ? __fdiv_rn(p[j], sum) : -1.0f;
    }
    for (int r = 0; r < topk; ++r) {
        float bv = -1.0f;
        int be = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = j * 32 + lane;
            if (p[j] > bv) { bv = p[j]; be = e; }    // ascending e per lane: first maximum wins
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        if (lane == 0) {
            inds[t * topk + r] = be;
            scores[t * topk + r] = f32_to_bf16(bv);
            if (scores_f32) scores_f32[t * topk + r] = bv;
        }
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (j * 32 + lane == be) p[j] = -1.0f;
    }
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_route_sort(const int32_t* inds, int64_t M, int topk, int E, int tm, int32_t* pos, int32_t* tok,
                               int32_t* esorted, int32_t* off, int32_t* tstart, void* stream) {
    SCMX_REQUIRE(M >= 0 && topk >= 1 && tm >= 1, SCMX_EINVAL, "route_sort: need M >= 0, topk >= 1, tm >= 1");
    SCMX_REQUIRE(E >= 1 && E <= 1024, SCMX_ELIMIT, "route_sort: E=%d outside 1..1024", E);
    SCMX_REQUIRE(M * topk < (1ll << 30), SCMX_ELIMIT, "route_sort: M*topk too large");
    const int R = (int)(M * topk);
    if (R >= 8192) {                     // a cluster of CTAs; below that one CTA finishes sooner than the cluster barriers cost
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(RS_CLUSTER);
        cfg.blockDim = dim3(1024);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = RS_CLUSTER;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_use_pdl ? 2 : 1;
        SCMX_PDL_OK("route_sort_cluster_kernel",
                    cudaLaunchKernelEx(&cfg, route_sort_cluster_kernel, inds, R, topk, E, tm, pos, tok, esorted, off, tstart));
        return SCMX_OK;
    }
    launch_pdl(route_sort_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, inds, R, topk, E, tm, pos, tok, esorted, off, tstart);
    SCMX_LAUNCH_OK("route_sort_kernel");
    return SCMX_OK;
}

extern "C" int scmx_router_topk(const float* logits, int64_t M, int E, int topk, int32_t* inds, uint16_t* scores,
                                float* scores_f32, void* stream) {
    SCMX_REQUIRE(M >= 0 && E >= 1 && E <= 1024 && topk >= 1 && topk <= E, SCMX_EINVAL,
                 "router_topk: need 1 <= topk <= E <= 1024 (E=%d topk=%d)", E, topk);
    if (M == 0) return SCMX_OK;
    const dim3 grid((unsigned)((M + 7) / 8)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    if (E <= 64) launch_pdl(router_topk_kernel<2>, grid, block, 0, st, logits, M, E, topk, inds, scores, scores_f32);
    else if (E <= 128) launch_pdl(router_topk_kernel<4>, grid, block, 0, st, logits, M, E, topk, inds, scores, scores_f32);
    else if (E <= 256) launch_pdl(router_topk_kernel<8>, grid, block, 0, st, logits, M, E, topk, inds, scores, scores_f32);
    else launch_pdl(router_topk_kernel<32>, grid, block, 0, st, logits, M, E, topk, inds, scores, scores_f32);
    SCMX_LAUNCH_OK("router_topk_kernel");
    return SCMX_OK;
}
