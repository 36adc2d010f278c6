// Expert-parallel token exchange over peer memory (NVLink), as kernels: no host round trip, no library collective, so a
// whole MoE half-block can be captured in a CUDA graph.
//
//   ep_dispatch   every sorted assignment row (INT8 activations + scale) is stored straight into the receive buffer of the
//                 GPU that owns its expert, at [source rank][position among the rows this source sends there]; the per-expert
//                 counts and the base row of that group in the source's sorted order travel with it.
//   peer_barrier  all GPUs signal each other through flag words in peer memory and wait (bounded) for everyone.
//   ep_plan       the receiver turns the count matrix [source][local expert] into expert segments (offsets, M-tile starts) and
//                 the gather list that regroups arrival order (source-major) into expert-major order, plus the return address
//                 (rank, row) of every regrouped row.
//   ep_return     expert outputs are stored back into the sender's buffer at the row they left from, so the sender's
//                 moe_combine finds them in its own sorted order.
//
// The reference is single-device; the order independence this relies on is the one it states for its own counting sort
// (e2e/sc_moe.py:110-113): every sorted row is computed independently.  All loads are plain loads of local memory; only
// stores cross NVLink.  Spin waits carry a wall-clock limit and report through a status word.
#include "scmx_common.cuh"
#include "scmx_ptx.cuh"

namespace scmx {

constexpr int MAX_PEERS = 8;

struct PeerPtrs {
    void* p[MAX_PEERS];
};

// One warp per row (eight rows in flight per CTA, four 16-byte loads per lane issued before the stores): a row's copy starts
// with three dependent index loads, which a CTA-per-row form exposes once per row.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs,
                                                          const int32_t* __restrict__ tok, const int32_t* __restrict__ esorted,
                                                          const int32_t* __restrict__ off, int R, int K, int E, int world, int rank,
                                                          int cap, PeerPtrs rx_q, PeerPtrs rx_s, PeerPtrs rx_meta) {
    pdl_launch_dependents();
    pdl_wait();
    const int El = E / world;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.x == gridDim.x - 1) {
        // the last CTA ships the count matrix: to rank d, the counts of its experts and the base row of that group here
        for (int i = threadIdx.x; i < world * (El + 1); i += blockDim.x) {
            const int d = i / (El + 1), le = i % (El + 1);
            const int v = le < El ? off[d * El + le + 1] - off[d * El + le] : off[d * El];
            reinterpret_cast<int32_t*>(rx_meta.p[d])[rank * (El + 1) + le] = v;
        }
    } else {
        const int nvec = K / 16;
        const int wstride = ((int)gridDim.x - 1) * 8;
        for (int p = (int)blockIdx.x * 8 + warp; p < R; p += wstride) {
            const int e = esorted[p];
            const int t = tok[p];
            const int d = e >= 0 ? e / El : world;
            if (d >= world || t < 0) continue;                                     // inconsistent routing tables: touch nothing
            const int idx = p - off[d * El];                 // position among the rows this rank sends to rank d
            if (idx < 0 || idx >= cap) continue;
            const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)t * K);
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<int8_t*>(rx_q.p[d]) + ((size_t)rank * cap + idx) * K);
            for (int i0 = lane; i0 < nvec; i0 += 128) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i0 + 32 * u < nvec) v[u] = src[i0 + 32 * u];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i0 + 32 * u < nvec) dst[i0 + 32 * u] = v[u];
            }
            if (lane == 0) reinterpret_cast<float*>(rx_s.p[d])[(size_t)rank * cap + idx] = xs[t];
        }
    }
    // one system-scope fence per CTA, after all of its threads' stores (the barrier kernel that follows publishes them)
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();
}

// flags: int32 [world] on every GPU; slot r of GPU g's array is written by rank r.  epoch lives on the local GPU.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, int32_t* epoch, int32_t* status, uint64_t limit_ns) {
    pdl_launch_dependents();
    pdl_wait();
    const int ep = *epoch + 1;
    if (threadIdx.x < world) {
        // release: everything this GPU wrote before (earlier kernels of the stream included) is visible system-wide before the flag
        int32_t* theirs = reinterpret_cast<int32_t*>(flags.p[threadIdx.x]) + rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(ep) : "memory");
        const int32_t* mine = reinterpret_cast<const int32_t*>(flags.p[rank]) + threadIdx.x;
        const uint64_t t0 = globaltimer_ns();
        for (;;) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v >= ep) break;
            if (globaltimer_ns() - t0 > limit_ns) {
                if (atomicCAS(status, 0, 20) == 0) { status[1] = rank; status[2] = threadIdx.x; }
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *epoch = ep;
}

__global__ void __launch_bounds__(1024) ep_plan_kernel(const int32_t* __restrict__ rx_meta, int world, int El, int cap, int tm,
                                                       int r_cap, int32_t* __restrict__ off2, int32_t* __restrict__ tstart2,
                                                       int32_t* __restrict__ tok2, int32_t* __restrict__ ret_rank,
                                                       int32_t* __restrict__ ret_row, int32_t* __restrict__ n_rows) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ int cnt[MAX_PEERS][128];
    __shared__ int src0[MAX_PEERS][128];      // first receive-buffer row of segment (s, le)
    __shared__ int dst0[MAX_PEERS][128];      // first regrouped row of segment (s, le)
    __shared__ int base[MAX_PEERS];
    __shared__ int s_off[129];
    const int tid = threadIdx.x;
    for (int i = tid; i < world * El; i += blockDim.x) cnt[i / El][i % El] = rx_meta[(i / El) * (El + 1) + (i % El)];
    if (tid < world) base[tid] = rx_meta[tid * (El + 1) + El];
    __syncthreads();
    if (tid < 32) {
        // exclusive scans over the local experts by one warp, 32 experts per round
        int o = 0, t = 0;
        for (int b0 = 0; b0 < El; b0 += 32) {
            const int le = b0 + tid;
            int c = 0;
            if (le < El)
                for (int s = 0; s < world; ++s) c += cnt[s][le];
            const int ti = (c + tm - 1) / tm;
            int so = c, st = ti;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int a = __shfl_up_sync(0xffffffffu, so, d), b = __shfl_up_sync(0xffffffffu, st, d);
                if (tid >= d) { so += a; st += b; }
            }
            if (le < El) { s_off[le] = o + so - c; off2[le] = o + so - c; tstart2[le] = t + st - ti; }
            o += __shfl_sync(0xffffffffu, so, 31);
            t += __shfl_sync(0xffffffffu, st, 31);
        }
        if (tid == 0) { s_off[El] = o; off2[El] = o; tstart2[El] = t; n_rows[0] = o; }
    }
    if (tid >= 32 && tid < 32 + world) {
        const int sidx = tid - 32;
        int a = sidx * cap;
        for (int le = 0; le < El; ++le) { src0[sidx][le] = a; a += cnt[sidx][le]; }
    }
    __syncthreads();
    for (int le = tid; le < El; le += blockDim.x) {
        int d = s_off[le];
        for (int s = 0; s < world; ++s) { dst0[s][le] = d; d += cnt[s][le]; }
    }
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
    for (int seg = warp; seg < world * El; seg += nwarp) {       // one warp per (source, local expert) segment
        const int s = seg / El, le = seg % El;
        const int c = cnt[s][le], a = src0[s][le], d = dst0[s][le];
        for (int i = lane; i < c; i += 32) {
            tok2[d + i] = a + i;
            ret_rank[d + i] = s;
            ret_row[d + i] = base[s] + (a + i - s * cap);
        }
    }
    const int total = s_off[El];
    for (int i = total + tid; i < total + tm && i < r_cap + tm; i += blockDim.x) tok2[i] = 0;   // padding rows (never stored)
}

__global__ void __launch_bounds__(128) ep_return_kernel(const uint16_t* __restrict__ y, const int32_t* __restrict__ ret_rank,
                                                        const int32_t* __restrict__ ret_row, const int32_t* __restrict__ n_rows, int D,
                                                        PeerPtrs y_back) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = n_rows[0];
    for (int p = blockIdx.x; p < n; p += gridDim.x) {
        const int rr = ret_rank[p], row = ret_row[p];
        if (rr < 0 || rr >= MAX_PEERS || y_back.p[rr] == nullptr || row < 0) continue;
        const uint4* src = reinterpret_cast<const uint4*>(y + (size_t)p * D);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y_back.p[rr]) + (size_t)row * D);
        for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();
}

// Row gather and activation quantization over a row count that lives on the device (rows beyond it are skipped; the tm rows
// right after it are zero-filled so that the last M tile of the grouped GEMM reads defined data).
// The grids of the two kernels below are bounded (a few CTAs per SM) and stride over the rows that exist: the capacity
// they are launched for is a worst case (every token of every rank routed here), the row count is known on the device only.
__global__ void __launch_bounds__(256) gather_rows_dyn_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs,
                                                              const int32_t* __restrict__ tok, const int32_t* __restrict__ n_rows, int pad,
                                                              int K, int8_t* __restrict__ dq, float* __restrict__ ds) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, n = n_rows[0], nv = K / 16;
    const int stride = gridDim.x * (blockDim.x >> 5);
    for (int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < n + pad; p += stride) {   // a warp per row
        uint4* dst = reinterpret_cast<uint4*>(dq + (size_t)p * K);
        if (p >= n) {
            for (int i = lane; i < nv; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const int t = tok[p];
        const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)t * K);
        for (int base = 0; base < nv; base += 32 * 8) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + j * 32 + lane;
                if (i < nv) v[j] = src[i];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + j * 32 + lane;
                if (i < nv) dst[i] = v[j];
            }
        }
        if (lane == 0) ds[p] = xs[t];
    }
}

__global__ void __launch_bounds__(256) act_quant_dyn_kernel(const uint16_t* __restrict__ x, const int32_t* __restrict__ n_rows, int pad,
                                                            int K, int8_t* __restrict__ xq, float* __restrict__ xs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int n = n_rows[0];
    for (int row = blockIdx.x; row < n + pad; row += gridDim.x) {     // uniform over the CTA: the barriers below are safe
    uint2* qrow = reinterpret_cast<uint2*>(xq + (size_t)row * K);
    if (row >= n) {
        for (int v = threadIdx.x; v < K / 8; v += blockDim.x) qrow[v] = make_uint2(0, 0);
        if (threadIdx.x == 0) xs[row] = 0.0f;
        continue;
    }
    const uint4* xrow = reinterpret_cast<const uint4*>(x + (size_t)row * K);
    float amax = 0.0f;
    for (int v = threadIdx.x; v < K / 8; v += blockDim.x) {
        const uint4 r = xrow[v];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
            amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xFFFF0000u))));
    }
    amax = block_max(amax, red);
    float s, qi;
    quant_scale(amax, s, qi);
    for (int v = threadIdx.x; v < K / 8; v += blockDim.x) {
        const uint4 r = xrow[v];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { f[2 * j] = __uint_as_float(w[j] << 16); f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u); }
        qrow[v] = make_uint2(quant4(f[0], f[1], f[2], f[3], qi), quant4(f[4], f[5], f[6], f[7], qi));
    }
    if (threadIdx.x == 0) xs[row] = s;
    }
}

// All-gather by stores: this rank's contiguous block is written at the same offset into every rank's buffer (its own
// included); a peer_barrier afterwards makes the gathered buffer complete everywhere.
__global__ void __launch_bounds__(256) peer_put_kernel(const uint4* __restrict__ src, int64_t n_vec, int64_t dst_off_vec, PeerPtrs dst) {
    pdl_launch_dependents();
    pdl_wait();
    uint4* out = reinterpret_cast<uint4*>(dst.p[blockIdx.y]) + dst_off_vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) out[i] = src[i];
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();
}

static int fill_peers(PeerPtrs* out, const void* const* host_ptrs, int world, const char* who) {
    SCMX_REQUIRE(world >= 1 && world <= MAX_PEERS, SCMX_ELIMIT, "%s: world=%d outside 1..%d", who, world, MAX_PEERS);
    for (int i = 0; i < MAX_PEERS; ++i) out->p[i] = i < world ? const_cast<void*>(host_ptrs[i]) : nullptr;
    for (int i = 0; i < world; ++i) SCMX_REQUIRE(out->p[i] != nullptr, SCMX_EINVAL, "%s: peer pointer %d is NULL", who, i);
    return SCMX_OK;
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_ep_dispatch(const int8_t* xq, const float* xs, const int32_t* tok, const int32_t* esorted, const int32_t* off,
                                int64_t R, int64_t K, int E, int world, int rank, int64_t cap, const void* const* rx_q_peers,
                                const void* const* rx_s_peers, const void* const* rx_meta_peers, void* stream) {
    PeerPtrs q, s, m;
    int rc = fill_peers(&q, rx_q_peers, world, "ep_dispatch");
    if (rc) return rc;
    if ((rc = fill_peers(&s, rx_s_peers, world, "ep_dispatch"))) return rc;
    if ((rc = fill_peers(&m, rx_meta_peers, world, "ep_dispatch"))) return rc;
    SCMX_REQUIRE(R >= 0 && R <= cap && K > 0 && K % 16 == 0 && E % world == 0 && E / world <= 128 && rank >= 0 && rank < world,
                 SCMX_EINVAL, "ep_dispatch: need R <= cap, K %% 16 == 0, E %% world == 0, E / world <= 128");
    const int64_t row_ctas = (R + 7) / 8;
    const unsigned dgrid = (unsigned)(row_ctas < 1184 ? row_ctas : 1184) + 1;     // warps loop over the rows; the last CTA ships the counts
    launch_pdl(ep_dispatch_kernel, dim3(dgrid), dim3(256), 0, (cudaStream_t)stream, xq, xs, tok, esorted, off, (int)R, (int)K,
               E, world, rank, (int)cap, q, s, m);
    SCMX_LAUNCH_OK("ep_dispatch_kernel");
    return SCMX_OK;
}

extern "C" int scmx_peer_barrier(const void* const* flag_peers, int rank, int world, int32_t* epoch, int32_t* status, void* stream) {
    PeerPtrs f;
    int rc = fill_peers(&f, flag_peers, world, "peer_barrier");
    if (rc) return rc;
    SCMX_REQUIRE(rank >= 0 && rank < world && epoch && status, SCMX_EINVAL, "peer_barrier: bad rank / epoch / status");
    launch_pdl(peer_barrier_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, f, rank, world, epoch, status, (uint64_t)g_wait_limit_ns);
    SCMX_LAUNCH_OK("peer_barrier_kernel");
    return SCMX_OK;
}

extern "C" int scmx_peer_put(const void* src, int64_t bytes, int64_t dst_offset_bytes, const void* const* dst_peers, int world,
                             void* stream) {
    PeerPtrs d;
    int rc = fill_peers(&d, dst_peers, world, "peer_put");
    if (rc) return rc;
    SCMX_REQUIRE(bytes >= 0 && bytes % 16 == 0 && dst_offset_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0, SCMX_EINVAL,
                 "peer_put: sizes, offsets and pointers must be multiples of 16 bytes");
    if (bytes == 0) return SCMX_OK;
    const int64_t n_vec = bytes / 16;
    int64_t blocks = (n_vec + 255) / 256;
    if (blocks > 296) blocks = 296;
    launch_pdl(peer_put_kernel, dim3((unsigned)blocks, (unsigned)world), dim3(256), 0, (cudaStream_t)stream,
               reinterpret_cast<const uint4*>(src), n_vec, dst_offset_bytes / 16, d);
    SCMX_LAUNCH_OK("peer_put_kernel");
    return SCMX_OK;
}

extern "C" int scmx_ep_plan(const int32_t* rx_meta, int world, int El, int64_t cap, int tm, int64_t r_cap, int32_t* off2,
                            int32_t* tstart2, int32_t* tok2, int32_t* ret_rank, int32_t* ret_row, int32_t* n_rows, void* stream) {
    SCMX_REQUIRE(world >= 1 && world <= MAX_PEERS && El >= 1 && El <= 128 && tm >= 1 && cap * world <= r_cap, SCMX_EINVAL,
                 "ep_plan: need world <= %d, El <= 128, world * cap <= r_cap", MAX_PEERS);
    launch_pdl(ep_plan_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, rx_meta, world, El, (int)cap, tm, (int)r_cap, off2, tstart2,
               tok2, ret_rank, ret_row, n_rows);
    SCMX_LAUNCH_OK("ep_plan_kernel");
    return SCMX_OK;
}

extern "C" int scmx_ep_return(const uint16_t* y, const int32_t* ret_rank, const int32_t* ret_row, const int32_t* n_rows, int64_t r_cap,
                              int64_t D, int world, const void* const* y_back_peers, void* stream) {
    PeerPtrs yb;
    int rc = fill_peers(&yb, y_back_peers, world, "ep_return");
    if (rc) return rc;
    SCMX_REQUIRE(r_cap >= 0 && D > 0 && D % 8 == 0, SCMX_EINVAL, "ep_return: D %% 8 != 0");
    if (r_cap == 0) return SCMX_OK;
    launch_pdl(ep_return_kernel, dim3((unsigned)(r_cap < 1184 ? r_cap : 1184)), dim3(128), 0, (cudaStream_t)stream, y, ret_rank, ret_row, n_rows, (int)D, yb);
    SCMX_LAUNCH_OK("ep_return_kernel");
    return SCMX_OK;
}

extern "C" int scmx_gather_rows_dyn(const int8_t* xq, const float* xs, const int32_t* tok, const int32_t* n_rows, int64_t r_cap, int pad,
                                    int64_t K, int8_t* dst_q, float* dst_s, void* stream) {
    SCMX_REQUIRE(r_cap >= 0 && pad >= 0 && K > 0 && K % 16 == 0, SCMX_EINVAL, "gather_rows_dyn: K %% 16 != 0");
    const int64_t g_ctas = (r_cap + pad + 7) / 8;
    launch_pdl(gather_rows_dyn_kernel, dim3((unsigned)(g_ctas < 148 * 8 ? g_ctas : 148 * 8)), dim3(256), 0, (cudaStream_t)stream, xq, xs, tok,
               n_rows, pad, (int)K, dst_q, dst_s);
    SCMX_LAUNCH_OK("gather_rows_dyn_kernel");
    return SCMX_OK;
}

extern "C" int scmx_act_quant_dyn(const uint16_t* x, const int32_t* n_rows, int64_t r_cap, int pad, int64_t K, int8_t* xq, float* xs,
                                  void* stream) {
    SCMX_REQUIRE(r_cap >= 0 && pad >= 0 && K > 0 && K % 8 == 0, SCMX_EINVAL, "act_quant_dyn: K %% 8 != 0");
    const int64_t a_ctas = r_cap + pad;
    launch_pdl(act_quant_dyn_kernel, dim3((unsigned)(a_ctas < 148 * 8 ? a_ctas : 148 * 8)), dim3(256), 0, (cudaStream_t)stream, x, n_rows, pad,
               (int)K, xq, xs);
    SCMX_LAUNCH_OK("act_quant_dyn_kernel");
    return SCMX_OK;
}

// Peer access from the current device to `peer_device` (needed before kernels dereference memory opened from another
// process's allocation on that device).  Already-enabled is not an error.
extern "C" int scmx_enable_peer_access(int peer_device) {
    int dev = 0;
    SCMX_CUDA_OK(cudaGetDevice(&dev));
    if (dev == peer_device) return SCMX_OK;
    int can = 0;
    SCMX_CUDA_OK(cudaDeviceCanAccessPeer(&can, dev, peer_device));
    SCMX_REQUIRE(can, SCMX_ECUDA, "device %d cannot access device %d over peer-to-peer", dev, peer_device);
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return SCMX_OK;
    }
    SCMX_CUDA_OK(e);
    return SCMX_OK;
}

