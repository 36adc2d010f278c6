// INT8 x INT8 -> INT32 GEMM for the W4A8 prefill path on sm_100a: tcgen05.mma kind::i8 with the accumulators in
// tensor memory, operands staged in shared memory by TMA, and the scaling epilogue fused.  One kernel serves the
// dense GEMM (xq [M,K] . wq [N,K]^T) and the grouped mixture-of-experts GEMM (row segments per expert).
//
// Persistent, warp-specialised CTA (one per SM, 320 threads):
//   warp 0      TMA producer: for every K block of 128 bytes loads a 128 x 128 tile of A and a BN x 128 tile of B into
//               one of STAGES shared-memory stages (128-byte swizzle), completing on the stage's "full" mbarrier.
//   warp 1      MMA issuer: one elected thread issues 4 tcgen05.mma (M128 x N BN x K32) per stage into one of two
//               TMEM accumulators (BN columns each), tcgen05.commit frees the stage ("empty" mbarrier) and, after the
//               last K block, publishes the accumulator ("tmem_full").  Also owns TMEM allocation.
//   warps 2..9  epilogue: each warp reads its 32 TMEM lanes x half of the tile's columns with tcgen05.ld (32 columns at a
//               time, the next load in flight while the current chunk is processed), applies
//               T((float(acc) * xscale[m]) * wscale[n]) (+ residual, or SwiGLU on interleaved gate/up columns) and
//               stores; then releases the accumulator ("tmem_empty") so the next tile's MMAs overlap this epilogue.
//
// Tiles are visited m-fastest inside bands of M tiles (get_tile) so that concurrently running CTAs share B tiles through L2.  No cluster launch: every CTA
// fetches its own tiles with its own TMA loads.  Every mbarrier wait is bounded by a wall-clock limit; when it runs
// out the kernel records where in `status`, lets in-flight copies land, frees its TMEM and returns.
#include "scmx_gemm_core.cuh"

namespace scmx {

// ---- the kernel -----------------------------------------------------------------------------------------------------------
template <int BN, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = BN * BK;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;                 // full[STAGES], empty[STAGES], tfull[2], tempty[2]
    static constexpr int MISC_OFF = BAR_OFF + 8 * (2 * STAGES + 4);      // tmem base (u32), abort flag (int)
    static constexpr int WS_OFF = MISC_OFF + 16;                         // wscale staging [2][BN] float
    static constexpr int EPI_OFF = WS_OFF + 2 * BN * 4;                  // epilogue staging, 16-byte aligned
    static constexpr int TOTAL = EPI_OFF + EPI_STAGE_BYTES + 1024;       // + slack for 1024-byte alignment
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(CTA_THREADS, 1) gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA,
                                                          const __grid_constant__ CUtensorMap tmB, const GemmArgs a) {
    using L = Smem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // stays a shared-space pointer
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + L::BAR_OFF, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC_OFF + 4);
    float* ws_stage = reinterpret_cast<float*>(smem + L::WS_OFF);
    constexpr uint32_t TMEM_COLS = 2 * BN;     // 256 or 512: a power of two >= 32

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, EPI_WARPS);      // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above (barrier init, TMEM allocation) overlapped the previous kernel's tail; operands, scales and
    // tile tables written by earlier kernels are only touched from here on
    pdl_wait();

    int tiles_m, slot0;
    const int total = num_tiles<BN>(a, tiles_m, slot0);
    const int num_kb = (a.K + BK - 1) / BK;
    int fail = 0;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = blockIdx.x; t < total && fail == 0; t += gridDim.x) {
                const Tile tl = get_tile<BN>(a, t, tiles_m, slot0);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (int w = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, a.wait_ns)) { fail = w == 1 ? 1 : -1; break; }
                    const uint32_t sa = sbase + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
                    mbar_expect_tx(bar_full + 8 * stage, L::STAGE_BYTES);
                    tma_load_2d(sa, &tmA, kb * BK, tl.row0, bar_full + 8 * stage);
                    tma_load_2d(sb, &tmB, kb * BK, tl.brow, bar_full + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            int stage = 0;
            uint32_t phase = 0, acc = 0, acc_phase = 0;
            for (int t = blockIdx.x; t < total && fail == 0; t += gridDim.x) {
                if (int w = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, a.wait_ns)) { fail = w == 1 ? 2 : -1; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (int w = mbar_wait(bar_full + 8 * stage, phase, abort_flag, a.wait_ns)) { fail = w == 1 ? 3 : -1; break; }
                    tc_fence_after();
                    const uint32_t sa = sbase + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
                    const uint64_t da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_i8(d_tmem, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc,
                                (kb | k) != 0 ? 1u : 0u);
                    umma_commit(bar_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (fail) break;
                umma_commit(bar_tfull + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------ epilogue warps 2..9: TMEM lane quarter = warp % 4 (the quarter
        // a warp may read), column half = (warp - 2) / 4.  Two warps per scheduler hide each other's latencies.
        const int q = warp & 3;
        const int chalf = (warp - 2) >> 2;
        const int et = threadIdx.x - 64;          // 0..255 among the epilogue threads
        uint32_t acc = 0, acc_phase = 0;
        for (int t = blockIdx.x; t < total && fail == 0; t += gridDim.x) {
            const Tile tl = get_tile<BN>(a, t, tiles_m, slot0);
            float* ws = ws_stage + acc * BN;
            if (a.epi != 0) {
                for (int i = et; i < BN; i += EPI_THREADS) ws[i] = (tl.n0 + i < a.N) ? a.wscale[tl.wrow + i] : 0.0f;
            }
            // what does not depend on the accumulators is fetched before they are awaited: the row's activation scale, the residual
            const int wrow0 = tl.row0 + 32 * q;
            const float xs = (a.epi != 0 && wrow0 + lane < tl.row_end) ? a.xscale[wrow0 + lane] : 0.0f;
            uint4 rp[8];
            if (a.epi == 2) epi_load_res(a, rp, lane, wrow0, tl.row_end, tl.n0 + chalf * (BN / 2));
            if (int w = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, a.wait_ns)) fail = w == 1 ? 4 : -1;
            // the epilogue threads agree on giving up (and see the staged scales) before anyone touches TMEM
            epilogue_bar();
            if (*abort_flag) { if (!fail) fail = -1; break; }
            tc_fence_after();
            epilogue_warp<BN>(a, tmem_base + acc * BN + chalf * (BN / 2) + ((uint32_t)(32 * q) << 16), ws + chalf * (BN / 2), wrow0,
                              tl.row_end, tl.n0 + chalf * (BN / 2), smem + L::EPI_OFF + (warp - 2) * EPI_STAGE_WARP, lane, xs, rp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }

    // status[0]: 1 producer waited for a free stage, 2 MMA waited for a free accumulator, 3 MMA waited for operands,
    // 4 epilogue waited for an accumulator; status[1] CTA, status[2] thread.  Secondary give-ups (fail < 0) are not recorded.
    if (fail > 0) {
        if (atomicCAS(a.status, 0, fail) == 0) {
            a.status[1] = blockIdx.x;
            a.status[2] = threadIdx.x;
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);   // 0.2 ms for outstanding TMA writes
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}


// ---- the same GEMM on CTA pairs (cta_group::2) ---------------------------------------------------------------------------
// Two CTAs on neighbouring SMs (a cluster of 2) share one 256 x 256 output tile.  Each CTA loads ITS 128 rows of A and ITS
// 128 of the tile's 256 weight rows (32 KB per K block instead of 48 KB for a 128 x 256 tile of its own), the leader CTA's MMA
// thread issues tcgen05.mma.cta_group::2 M256 x N256 x K32, which reads both CTAs' shared memory and writes 128 accumulator
// rows into each CTA's tensor memory, and each CTA runs the epilogue of its own 128 rows.  Operand bytes per MMA cycle drop by
// a third, which is what bounds the single-CTA kernel (its TMA stages arrive slower than the tensor core consumes them).
//   full[s]   lives in the leader: armed by the leader's producer for both CTAs' bytes; the peer's TMA loads complete on it
//             through the .cta_group::2 form of the copy (no multicast: every CTA fetches its own tiles)
//   empty[s], tmem_full[acc]   one copy per CTA, signalled in both CTAs by the leader's tcgen05.commit (multicast arrive)
//   tmem_empty[acc]            lives in the leader: 8 epilogue warps of each CTA arrive (the peer's remotely)
// Both CTAs meet at a cluster barrier after set-up and before tear-down, so neither touches the other's shared memory or
// tensor memory outside that window.  Waits are bounded as in the single-CTA kernel.
constexpr int PAIR_STAGES = 5;
constexpr int PAIR_BN = 256;
struct PairSmem {
    static constexpr int A_BYTES = BM * BK;                 // this CTA's 128 rows of the 256-row A tile
    static constexpr int B_BYTES = (PAIR_BN / 2) * BK;      // this CTA's 128 of the tile's 256 weight rows
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFF = PAIR_STAGES * STAGE_BYTES;
    static constexpr int MISC_OFF = BAR_OFF + 8 * (2 * PAIR_STAGES + 4);
    static constexpr int WS_OFF = MISC_OFF + 16;
    static constexpr int EPI_OFF = WS_OFF + 2 * PAIR_BN * 4;
    static constexpr int TOTAL = EPI_OFF + EPI_STAGE_BYTES + 1024;
};

// BCAST: the tensor-parallel form whose epilogue stores every output line into all ranks' buffers (a.bcast of them); an
// instantiation of its own so that the ordinary kernel's drain loop carries none of it.
template <bool BCAST>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(CTA_THREADS, 1)
    gemm_i8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs a) {
    using L = PairSmem;
    constexpr int STAGES = PAIR_STAGES, BN = PAIR_BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + L::BAR_OFF, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC_OFF + 4);
    float* ws_stage = reinterpret_cast<float*>(smem + L::WS_OFF);
    constexpr uint32_t TMEM_COLS = 2 * BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 2 * EPI_WARPS);      // the epilogue warps of both CTAs
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
    cluster_sync_all();             // the peer's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    const uint32_t full_leader = mapa_u32(bar_full, 0), tempty_leader = mapa_u32(bar_tempty, 0);
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int tiles_m = (a.M + 2 * BM - 1) / (2 * BM), tiles_n = (a.N + BN - 1) / BN;
    const int total = tiles_m * tiles_n;
    const int num_kb = (a.K + BK - 1) / BK;
    int fail = 0;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = pair; t < total && fail == 0; t += npairs) {
                const int nt = t / tiles_m, mt = t - nt * tiles_m;
                const int row0 = mt * 2 * BM + (int)rank * BM, brow = nt * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (int w = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, a.wait_ns)) { fail = w == 1 ? 1 : -1; break; }
                    const uint32_t sa = sbase + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
                    if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * L::STAGE_BYTES);
                    tma_load_2d_pair(sa, &tmA, kb * BK, row0, full_leader + 8 * stage);
                    tma_load_2d_pair(sb, &tmB, kb * BK, brow, full_leader + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc(2 * BM, BN);
            int stage = 0;
            uint32_t phase = 0, acc = 0, acc_phase = 0;
            for (int t = pair; t < total && fail == 0; t += npairs) {
                if (int w = mbar_wait_cluster(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, a.wait_ns)) { fail = w == 1 ? 2 : -1; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (int w = mbar_wait(bar_full + 8 * stage, phase, abort_flag, a.wait_ns)) { fail = w == 1 ? 3 : -1; break; }
                    tc_fence_after();
                    const uint32_t sa = sbase + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
                    const uint64_t da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_i8_pair(d_tmem, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc,
                                     (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(bar_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (fail) break;
                umma_commit_pair(bar_tfull + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        const int q = warp & 3;
        const int chalf = (warp - 2) >> 2;
        const int et = threadIdx.x - 64;
        uint32_t acc = 0, acc_phase = 0;
        for (int t = pair; t < total && fail == 0; t += npairs) {
            const int nt = t / tiles_m, mt = t - nt * tiles_m;
            const int n0 = nt * BN, row0 = mt * 2 * BM + (int)rank * BM;
            float* ws = ws_stage + acc * BN;
            if (a.epi != 0) {
                for (int i = et; i < BN; i += EPI_THREADS) ws[i] = (n0 + i < a.N) ? a.wscale[n0 + i] : 0.0f;
            }
            const int wrow0 = row0 + 32 * q;
            const float xs = (a.epi != 0 && wrow0 + lane < a.M) ? a.xscale[wrow0 + lane] : 0.0f;
            uint4 rp[8];
            if (a.epi == 2) epi_load_res(a, rp, lane, wrow0, a.M, n0 + chalf * (BN / 2));
            if (int w = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, a.wait_ns)) fail = w == 1 ? 4 : -1;
            epilogue_bar();
            if (*abort_flag) { if (!fail) fail = -1; break; }
            tc_fence_after();
            epilogue_warp<BN, true, BCAST>(a, tmem_base + acc * BN + chalf * (BN / 2) + ((uint32_t)(32 * q) << 16), ws + chalf * (BN / 2),
                                           wrow0, a.M, n0 + chalf * (BN / 2), smem + L::EPI_OFF + (warp - 2) * EPI_STAGE_WARP, lane, xs, rp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(bar_tempty + 8 * acc);
                else mbar_arrive_cluster(tempty_leader + 8 * acc);
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }

    if (fail > 0) {
        if (atomicCAS(a.status, 0, fail) == 0) {
            a.status[1] = blockIdx.x;
            a.status[2] = threadIdx.x;
        }
    }
    if (BCAST && warp >= 2) __threadfence_system();      // this thread's stores into the peers' buffers are performed
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);   // 0.2 ms for outstanding TMA writes
        __syncthreads();
    }
    cluster_sync_all();             // both CTAs are done with each other's shared and tensor memory
    tc_fence_after();
    if (warp == 1) tmem_dealloc2(tmem_base, TMEM_COLS);
}


// ---- SiLU table for the SwiGLU epilogue ----------------------------------------------------------------------------------
// silu(g) = T(g * sigmoid_T(g)) depends on the bf16 gate alone, so the epilogue reads it from a table with one entry per bf16
// bit pattern.  The table is filled on the device by the same step-by-step bf16 formula the row kernels use.
__device__ __align__(256) uint16_t g_silu_lut[65536];

__global__ void silu_lut_init_kernel() {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 65536u) g_silu_lut[i] = f32_to_bf16(silu_bf16(bf16_to_f32((uint16_t)i)));
}

// Device address of the table for the current device; built on the first call per device (stream-ordered on `st`, followed
// by one synchronisation of that stream so that later calls on other streams see it).
int silu_lut_ptr(cudaStream_t st, const uint16_t** out) {
    static const uint16_t* ptrs[64] = {};
    int dev = 0;
    SCMX_CUDA_OK(cudaGetDevice(&dev));
    SCMX_REQUIRE(dev >= 0 && dev < 64, SCMX_ELIMIT, "device ordinal %d out of range", dev);
    if (!ptrs[dev]) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        SCMX_CUDA_OK(cudaStreamIsCapturing(st, &cap));
        SCMX_REQUIRE(cap == cudaStreamCaptureStatusNone, SCMX_EINVAL,
                     "the first SwiGLU-epilogue GEMM on a device builds a table: call it once outside stream capture");
        void* p = nullptr;
        SCMX_CUDA_OK(cudaGetSymbolAddress(&p, g_silu_lut));
        silu_lut_init_kernel<<<256, 256, 0, st>>>();
        SCMX_LAUNCH_OK("silu_lut_init_kernel");
        SCMX_CUDA_OK(cudaStreamSynchronize(st));
        ptrs[dev] = static_cast<const uint16_t*>(p);
    }
    *out = ptrs[dev];
    return SCMX_OK;
}

// ---- host side ------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Byte matrix [rows, row_bytes] row-major, box = box_bytes x box_rows, swizzle of 128 or 64 bytes, zero fill outside.
int make_map_u8(CUtensorMap* map, const void* ptr, int64_t rows, int64_t row_bytes, int box_bytes, int box_rows, int swizzle_bytes) {
    EncodeTiledFn fn = encode_fn();
    SCMX_REQUIRE(fn != nullptr, SCMX_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SCMX_REQUIRE(r == CUDA_SUCCESS, SCMX_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld row_bytes=%lld)", (int)r,
                 (long long)rows, (long long)row_bytes);
    return SCMX_OK;
}
// INT8 operand [rows, K]: box = 128 bytes of K x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows) {
    return make_map_u8(map, ptr, rows, K, BK, box_rows, 128);
}

static int g_bn_override = 0;      // 0 = choose per problem
static int g_use_pair = 1;         // dense GEMMs of at least 256 x 256 run on CTA pairs
static int num_sms() { return sm_count(); }

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, int grid, cudaStream_t st) {
    using L = Smem<BN, STAGES>;
    static bool configured[64] = {};      // the attribute belongs to the current device's copy of the kernel
    const int dev = current_device();
    SCMX_REQUIRE(dev >= 0, SCMX_ECUDA, "no current CUDA device (ordinal 0..63)");
    if (!configured[dev]) {
        SCMX_CUDA_OK(cudaFuncSetAttribute(gemm_i8_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        configured[dev] = true;
    }
    launch_pdl(gemm_i8_kernel<BN, STAGES>, dim3(grid), dim3(CTA_THREADS), (size_t)L::TOTAL, st, tmA, tmB, a);
    SCMX_LAUNCH_OK("gemm_i8_kernel");
    return SCMX_OK;
}

static int run_gemm(const int8_t* xq, int64_t a_rows, const int8_t* wq, int64_t b_rows, GemmArgs& a, cudaStream_t st) {
    int bn = g_bn_override ? g_bn_override : (a.N >= 256 ? 256 : 128);
    a.wait_ns = g_wait_limit_ns;
    if (a.epi == 3) {
        int rc3 = silu_lut_ptr(st, &a.silu_lut);
        if (rc3) return rc3;
    }
    CUtensorMap tmA, tmB;
    int rc = make_map(&tmA, xq, a_rows, a.K, BM);
    if (rc) return rc;
    if (a.E == 0 && g_use_pair && !g_bn_override && a.M > BM && a.N >= PAIR_BN && a.ret_rank == nullptr) {
        rc = make_map(&tmB, wq, b_rows, a.K, PAIR_BN / 2);
        if (rc) return rc;
        const int64_t tiles = ((a.M + 2 * BM - 1) / (2 * BM)) * (int64_t)((a.N + PAIR_BN - 1) / PAIR_BN);
        int pairs = num_sms() / 2;
        if (tiles < pairs) pairs = (int)tiles;
        static bool configured[64] = {};
        const int dev = current_device();
        SCMX_REQUIRE(dev >= 0, SCMX_ECUDA, "no current CUDA device (ordinal 0..63)");
        if (!configured[dev]) {
            SCMX_CUDA_OK(cudaFuncSetAttribute(gemm_i8_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL));
            SCMX_CUDA_OK(cudaFuncSetAttribute(gemm_i8_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL));
            configured[dev] = true;
        }
        if (a.bcast > 0)
            SCMX_PDL_OK("gemm_i8_pair_kernel", launch_pdl(gemm_i8_pair_kernel<true>, dim3(2 * pairs), dim3(CTA_THREADS), (size_t)PairSmem::TOTAL, st, tmA, tmB, a));
        else
            SCMX_PDL_OK("gemm_i8_pair_kernel", launch_pdl(gemm_i8_pair_kernel<false>, dim3(2 * pairs), dim3(CTA_THREADS), (size_t)PairSmem::TOTAL, st, tmA, tmB, a));
        return SCMX_OK;
    }
    rc = make_map(&tmB, wq, b_rows, a.K, bn);
    if (rc) return rc;
    int grid = num_sms();
    if (a.E == 0) {
        const int64_t tiles = ((a.M + BM - 1) / BM) * (int64_t)((a.N + bn - 1) / bn);
        if (tiles < grid) grid = (int)tiles;
    }
    if (bn == 256) return launch_gemm<256, 3>(tmA, tmB, a, grid, st);
    return launch_gemm<128, 5>(tmA, tmB, a, grid, st);
}

// A per-device side stream and the events that order it against the caller's stream (created on first use; event waits and
// records are legal during stream capture, where they become graph dependencies).
struct SideStream {
    cudaStream_t side;
    cudaEvent_t fork, decoded[2], gemm_done[2];
};
static int side_stream(SideStream** out) {
    static SideStream ctx[64];
    static bool ready[64] = {};
    int dev = 0;
    SCMX_CUDA_OK(cudaGetDevice(&dev));
    SCMX_REQUIRE(dev >= 0 && dev < 64, SCMX_ELIMIT, "device ordinal %d out of range", dev);
    if (!ready[dev]) {
        SCMX_CUDA_OK(cudaStreamCreateWithFlags(&ctx[dev].side, cudaStreamNonBlocking));
        cudaEvent_t* ev[5] = {&ctx[dev].fork, &ctx[dev].decoded[0], &ctx[dev].decoded[1], &ctx[dev].gemm_done[0], &ctx[dev].gemm_done[1]};
        for (int i = 0; i < 5; ++i) SCMX_CUDA_OK(cudaEventCreateWithFlags(ev[i], cudaEventDisableTiming));
        ready[dev] = true;
    }
    *out = &ctx[dev];
    return SCMX_OK;
}

int check_common(const char* who, int64_t N, int64_t K, int epi, const float* xscale, const float* wscale,
                        const void* out, const int32_t* status) {
    SCMX_REQUIRE(N > 0 && N % 32 == 0 && N < (1ll << 30), SCMX_EINVAL, "%s: N=%lld must be a positive multiple of 32", who,
                 (long long)N);
    SCMX_REQUIRE(K > 0 && K % 16 == 0 && K < (1ll << 30), SCMX_EINVAL, "%s: K=%lld must be a positive multiple of 16", who,
                 (long long)K);
    SCMX_REQUIRE(epi >= 0 && epi <= 3, SCMX_EINVAL, "%s: epi=%d outside 0..3", who, epi);
    SCMX_REQUIRE(epi == 0 || (xscale && wscale), SCMX_EINVAL, "%s: epi %d needs xscale and wscale", who, epi);
    SCMX_REQUIRE(out && status, SCMX_EINVAL, "%s: out / status is NULL", who);
    SCMX_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15) == 0, SCMX_EINVAL, "%s: out must be 16-byte aligned", who);
    SCMX_REQUIRE(epi != 3 || N % 64 == 0, SCMX_EINVAL, "%s: epi 3 needs N %% 64 == 0", who);
    return SCMX_OK;
}

}  // namespace scmx

using namespace scmx;

extern "C" int scmx_set_gemm_pair(int enable) {
    g_use_pair = enable ? 1 : 0;
    return SCMX_OK;
}

extern "C" int scmx_set_gemm_tile(int bn) {
    SCMX_REQUIRE(bn == 0 || bn == 128 || bn == 256, SCMX_EINVAL, "set_gemm_tile: bn=%d (0 = automatic, 128 or 256)", bn);
    g_bn_override = bn;
    return SCMX_OK;
}

extern "C" int scmx_mm_i8(const int8_t* xq, const int8_t* wq, int64_t M, int64_t N, int64_t K, int epi, const float* xscale,
                          const float* wscale, const uint16_t* res, void* out, int32_t* status, void* stream) {
    int rc = check_common("mm_i8", N, K, epi, xscale, wscale, out, status);
    if (rc) return rc;
    SCMX_REQUIRE(M >= 0 && M < (1ll << 30), SCMX_EINVAL, "mm_i8: M=%lld out of range", (long long)M);
    SCMX_REQUIRE(epi != 2 || res, SCMX_EINVAL, "mm_i8: epi 2 needs res");
    SCMX_REQUIRE((reinterpret_cast<uintptr_t>(xq) & 15) == 0 && (reinterpret_cast<uintptr_t>(wq) & 15) == 0 &&
                     (!res || (reinterpret_cast<uintptr_t>(res) & 15) == 0),
                 SCMX_EINVAL, "mm_i8: xq, wq and res must be 16-byte aligned");
    if (M == 0) return SCMX_OK;
    GemmArgs a = {};
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.epi = epi; a.xscale = xscale; a.wscale = wscale; a.res = res; a.out = out;
    a.status = status;
    return run_gemm(xq, M, wq, N, a, (cudaStream_t)stream);
}

extern "C" int scmx_mm_i8_bcast(const int8_t* xq, const int8_t* wq, int64_t M, int64_t N, int64_t K, int epi, const float* xscale,
                                const float* wscale, const uint16_t* res, void* const* out_peers, int world, int32_t* status,
                                void* stream) {
    int rc = check_common("mm_i8_bcast", N, K, epi, xscale, wscale, out_peers, status);
    if (rc) return rc;
    SCMX_REQUIRE(epi >= 1 && epi <= 3, SCMX_EINVAL, "mm_i8_bcast: epi must be 1, 2 or 3");
    SCMX_REQUIRE(M > BM && M < (1ll << 30) && N >= PAIR_BN, SCMX_ELIMIT, "mm_i8_bcast: needs M > %d and N >= %d (the CTA-pair kernel)", BM, PAIR_BN);
    SCMX_REQUIRE(epi != 2 || res, SCMX_EINVAL, "mm_i8_bcast: epi 2 needs res");
    SCMX_REQUIRE(world >= 1 && world <= 8, SCMX_EINVAL, "mm_i8_bcast: world=%d outside 1..8", world);
    SCMX_REQUIRE((reinterpret_cast<uintptr_t>(xq) & 15) == 0 && (reinterpret_cast<uintptr_t>(wq) & 15) == 0 &&
                     (!res || (reinterpret_cast<uintptr_t>(res) & 15) == 0),
                 SCMX_EINVAL, "mm_i8_bcast: xq, wq and res must be 16-byte aligned");
    GemmArgs a = {};
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.epi = epi; a.xscale = xscale; a.wscale = wscale; a.res = res; a.out = out_peers[0];
    a.status = status; a.bcast = world;
    for (int g = 0; g < 8; ++g) {
        a.peer_out[g] = g < world ? static_cast<uint16_t*>(out_peers[g]) : nullptr;
        SCMX_REQUIRE(g >= world || (a.peer_out[g] != nullptr && (reinterpret_cast<uintptr_t>(a.peer_out[g]) & 15) == 0), SCMX_EINVAL,
                     "mm_i8_bcast: output buffer of rank %d is NULL or not 16-byte aligned", g);
    }
    SCMX_REQUIRE(g_use_pair && !g_bn_override, SCMX_EINVAL, "mm_i8_bcast: the CTA-pair kernel is switched off");
    return run_gemm(xq, M, wq, N, a, (cudaStream_t)stream);
}

extern "C" int scmx_moe_mm_i8(const int8_t* xq, int64_t R, const int8_t* wq, const float* wscale, const int32_t* off,
                              const int32_t* tstart, int E, int64_t N, int64_t K, int epi, const float* xscale, void* out,
                              int tm, int32_t* status, void* stream) {
    int rc = check_common("moe_mm_i8", N, K, epi, xscale, wscale, out, status);
    if (rc) return rc;
    SCMX_REQUIRE(epi != 2, SCMX_EINVAL, "moe_mm_i8: epi must be 0, 1 or 3");
    SCMX_REQUIRE(tm == BM, SCMX_EINVAL, "moe_mm_i8: tm=%d, the kernel's M tile is %d (pass tm=%d to route_sort)", tm, BM, BM);
    SCMX_REQUIRE(E >= 1 && E <= 65536 && R >= 0 && R < (1ll << 30) && off && tstart, SCMX_EINVAL, "moe_mm_i8: bad E / R / offsets");
    SCMX_REQUIRE((int64_t)E * N < (1ll << 31), SCMX_ELIMIT, "moe_mm_i8: E*N too large");
    if (R == 0) return SCMX_OK;
    GemmArgs a = {};
    a.M = (int)R; a.N = (int)N; a.K = (int)K; a.epi = epi; a.xscale = xscale; a.wscale = wscale; a.out = out;
    a.off = off; a.tstart = tstart; a.E = E; a.e_begin = 0; a.e_end = E; a.status = status;
    return run_gemm(xq, R, wq, (int64_t)E * N, a, (cudaStream_t)stream);
}

extern "C" int scmx_moe_mm_i8_ret(const int8_t* xq, int64_t R, const int8_t* wq, const float* wscale, const int32_t* off,
                                  const int32_t* tstart, int E, int64_t N, int64_t K, const float* xscale, const int32_t* ret_rank,
                                  const int32_t* ret_row, int world, void* const* out_peers, int tm, int32_t* status,
                                  void* stream) {
    int rc = check_common("moe_mm_i8_ret", N, K, 1, xscale, wscale, out_peers, status);
    if (rc) return rc;
    SCMX_REQUIRE(tm == BM, SCMX_EINVAL, "moe_mm_i8_ret: tm=%d, the kernel's M tile is %d", tm, BM);
    SCMX_REQUIRE(E >= 1 && E <= 65536 && R >= 0 && R < (1ll << 30) && off && tstart, SCMX_EINVAL, "moe_mm_i8_ret: bad E / R / offsets");
    SCMX_REQUIRE((int64_t)E * N < (1ll << 31), SCMX_ELIMIT, "moe_mm_i8_ret: E*N too large");
    SCMX_REQUIRE(ret_rank && ret_row && world >= 1 && world <= 8, SCMX_EINVAL, "moe_mm_i8_ret: return map / world (1..8)");
    if (R == 0) return SCMX_OK;
    GemmArgs a = {};
    a.M = (int)R; a.N = (int)N; a.K = (int)K; a.epi = 1; a.xscale = xscale; a.wscale = wscale; a.out = out_peers[0];
    a.off = off; a.tstart = tstart; a.E = E; a.e_begin = 0; a.e_end = E; a.status = status;
    a.ret_rank = ret_rank; a.ret_row = ret_row;
    for (int g = 0; g < 8; ++g) {
        a.peer_out[g] = g < world ? static_cast<uint16_t*>(out_peers[g]) : nullptr;
        SCMX_REQUIRE(g >= world || (a.peer_out[g] != nullptr && (reinterpret_cast<uintptr_t>(a.peer_out[g]) & 15) == 0), SCMX_EINVAL,
                     "moe_mm_i8_ret: return buffer of rank %d is NULL or not 16-byte aligned", g);
    }
    return run_gemm(xq, R, wq, (int64_t)E * N, a, (cudaStream_t)stream);
}

extern "C" int scmx_moe_mm(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                           const int32_t* off, const int32_t* tstart, int E, int64_t N, int64_t K, const scmx_format* fmt,
                           int epi, const float* xscale, void* out, int tm, int experts_per_pass, int8_t* scratch,
                           int64_t scratch_bytes, int32_t* status, void* stream) {
    int rc = check_common("moe_mm", N, K, epi, xscale, wscale, out, status);
    if (rc) return rc;
    DevFormat f;
    rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    SCMX_REQUIRE(epi != 2, SCMX_EINVAL, "moe_mm: epi must be 0, 1 or 3");
    SCMX_REQUIRE(tm == BM, SCMX_EINVAL, "moe_mm: tm=%d, the kernel's M tile is %d (pass tm=%d to route_sort)", tm, BM, BM);
    SCMX_REQUIRE(E >= 1 && E <= 65536 && R >= 0 && R < (1ll << 30) && off && tstart, SCMX_EINVAL, "moe_mm: bad E / R / offsets");
    SCMX_REQUIRE(experts_per_pass >= 1, SCMX_EINVAL, "moe_mm: experts_per_pass must be >= 1");
    const int64_t half = (int64_t)experts_per_pass * N * K;
    SCMX_REQUIRE(scratch && scratch_bytes >= 2 * half, SCMX_EINVAL,
                 "moe_mm: scratch of %lld bytes is smaller than 2 * experts_per_pass * N * K = %lld", (long long)scratch_bytes,
                 (long long)(2 * half));
    SCMX_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 1023) == 0, SCMX_EINVAL, "moe_mm: scratch must be 1024-byte aligned");
    if (R == 0) return SCMX_OK;
    const int64_t wpe = N * K / 8;                              // code words per expert
    const int64_t bpe = N * (K / (f.block * f.blocks_per_byte));  // block-code bytes per expert
    cudaStream_t main_s = (cudaStream_t)stream;
    SideStream* sd = nullptr;
    rc = side_stream(&sd);
    if (rc) return rc;
    const int passes = (E + experts_per_pass - 1) / experts_per_pass;
    // The decode of pass p+1 runs on a side stream while the GEMM of pass p runs on the caller's stream; two scratch
    // halves alternate, so the decode of pass p+1 also waits for the GEMM of pass p-1 (the last reader of its half).
    auto decode = [&](int p, cudaStream_t st) -> int {
        const int e0 = p * experts_per_pass;
        const int e1 = e0 + experts_per_pass < E ? e0 + experts_per_pass : E;
        return scmx_unpack_i8(codes + e0 * wpe, bcodes + e0 * bpe, (int64_t)(e1 - e0) * N, K, fmt, scratch + (p & 1) * half, st);
    };
    SCMX_CUDA_OK(cudaEventRecord(sd->fork, main_s));
    SCMX_CUDA_OK(cudaStreamWaitEvent(sd->side, sd->fork, 0));
    rc = decode(0, sd->side);
    if (rc) return rc;
    SCMX_CUDA_OK(cudaEventRecord(sd->decoded[0], sd->side));
    for (int p = 0; p < passes; ++p) {
        if (p + 1 < passes) {
            if (p >= 1) SCMX_CUDA_OK(cudaStreamWaitEvent(sd->side, sd->gemm_done[(p - 1) & 1], 0));
            rc = decode(p + 1, sd->side);
            if (rc) return rc;
            SCMX_CUDA_OK(cudaEventRecord(sd->decoded[(p + 1) & 1], sd->side));
        }
        SCMX_CUDA_OK(cudaStreamWaitEvent(main_s, sd->decoded[p & 1], 0));
        const int e0 = p * experts_per_pass;
        const int e1 = e0 + experts_per_pass < E ? e0 + experts_per_pass : E;
        GemmArgs a = {};
        a.M = (int)R; a.N = (int)N; a.K = (int)K; a.epi = epi; a.xscale = xscale; a.wscale = wscale; a.out = out;
        a.off = off; a.tstart = tstart; a.E = E; a.e_begin = e0; a.e_end = e1; a.status = status;
        rc = run_gemm(xq, R, scratch + (p & 1) * half, (int64_t)(e1 - e0) * N, a, main_s);
        if (rc) return rc;
        SCMX_CUDA_OK(cudaEventRecord(sd->gemm_done[p & 1], main_s));
    }
    return SCMX_OK;
}

// ---- grouped GEMM from packed weights with the scratch held inside the library ------------------------------------------
// Some hosts of this library cannot give it scratch memory: a serving process that hands all of HBM to its own
// KV-cache / activation pool at start-up has nothing left to cudaMalloc from later (and cudaMalloc would stall the device
// in the middle of a request), and a runtime that binds the C ABI from another language often has no device allocator
// at all.  For them the decoded-INT8 staging area of the grouped GEMM lives in this fixed array: two halves of 8 MiB,
// resident on every GPU that loads the library until the process exits.
namespace scmx {
constexpr int64_t MOE_STATIC_HALF_BYTES = 8ll << 20;
static __device__ __align__(256) int8_t g_moe_static_scratch[2 * MOE_STATIC_HALF_BYTES];

// The array's name is only a host-side handle; kernels need its device address, looked up once per device with that
// device current.
static int moe_static_scratch_ptr(cudaStream_t st, int8_t** out) {
    static int8_t* ptrs[64] = {};
    int dev = 0;
    SCMX_CUDA_OK(cudaGetDevice(&dev));
    SCMX_REQUIRE(dev >= 0 && dev < 64, SCMX_ELIMIT, "device ordinal %d out of range", dev);
    if (!ptrs[dev]) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        SCMX_CUDA_OK(cudaStreamIsCapturing(st, &cap));
        SCMX_REQUIRE(cap == cudaStreamCaptureStatusNone, SCMX_EINVAL,
                     "moe_mm_static: the first call on a device looks up the built-in scratch; make it outside stream capture");
        int8_t* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_moe_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("cudaGetSymbolAddress(g_moe_static_scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
            return SCMX_ECUDA;
        }
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return SCMX_OK;
}
}  // namespace scmx

extern "C" int scmx_moe_mm_static(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes,
                                  const float* wscale, const int32_t* off, const int32_t* tstart, int E, int64_t N, int64_t K,
                                  const scmx_format* fmt, int epi, const float* xscale, void* out, int tm, int32_t* status,
                                  void* stream) {
    int rc = check_common("moe_mm_static", N, K, epi, xscale, wscale, out, status);
    if (rc) return rc;
    DevFormat f;
    rc = make_dev_format(fmt, &f);
    if (rc) return rc;
    SCMX_REQUIRE(epi != 2, SCMX_EINVAL, "moe_mm_static: epi must be 0, 1 or 3");
    SCMX_REQUIRE(tm == BM, SCMX_EINVAL, "moe_mm_static: tm=%d, the kernel's M tile is %d (pass tm=%d to route_sort)", tm, BM, BM);
    SCMX_REQUIRE(E >= 1 && E <= 65536 && R >= 0 && R < (1ll << 30) && off && tstart, SCMX_EINVAL,
                 "moe_mm_static: bad E / R / offsets");
    SCMX_REQUIRE(N * K <= MOE_STATIC_HALF_BYTES, SCMX_ELIMIT,
                 "moe_mm_static: one decoded expert matrix is N*K = %lld bytes, more than the %lld bytes of one half of the "
                 "built-in scratch; use scmx_moe_mm with caller-provided scratch",
                 (long long)(N * K), (long long)MOE_STATIC_HALF_BYTES);
    if (R == 0) return SCMX_OK;
    int8_t* scratch = nullptr;
    rc = moe_static_scratch_ptr((cudaStream_t)stream, &scratch);
    if (rc) return rc;
    const int epp = (int)(MOE_STATIC_HALF_BYTES / (N * K));      // experts decoded per pass (>= 1)
    const int64_t half = MOE_STATIC_HALF_BYTES;
    const int64_t wpe = N * K / 8;
    const int64_t bpe = N * (K / (f.block * f.blocks_per_byte));
    int pass = 0;
    for (int e0 = 0; e0 < E; e0 += epp, ++pass) {
        const int e1 = e0 + epp < E ? e0 + epp : E;
        int8_t* buf = scratch + (pass & 1) * half;
        // every byte the GEMM reads from `buf` is rewritten here first, so nothing left by an earlier call is ever used
        rc = scmx_unpack_i8(codes + e0 * wpe, bcodes + e0 * bpe, (int64_t)(e1 - e0) * N, K, fmt, buf, stream);
        if (rc) return rc;
        GemmArgs a = {};
        a.M = (int)R; a.N = (int)N; a.K = (int)K; a.epi = epi; a.xscale = xscale; a.wscale = wscale; a.out = out;
        a.off = off; a.tstart = tstart; a.E = E; a.e_begin = e0; a.e_end = e1; a.status = status;
        rc = run_gemm(xq, R, buf, (int64_t)(e1 - e0) * N, a, (cudaStream_t)stream);
        if (rc) return rc;
    }
    return SCMX_OK;
}

