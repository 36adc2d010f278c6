/* scmx.h — C ABI of libscmx.so: the SC-MXFP4 W4A8 hot path on NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer.  Nothing is allocated or freed across the ABI: outputs and scratch
 *     buffers are preallocated by the caller.
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and nothing synchronises.
 *   - Return value: 0 on success, a negative SCMX_E* code otherwise; scmx_last_error_string() describes the last
 *     failure on the calling thread.  Shapes are validated on the host before anything is launched.
 *   - Matrices are row-major; weights are [N, K] (out_features, in_features) with K contiguous, activations [M, K].
 *   - "bf16" buffers hold bfloat16 bit patterns (uint16_t).
 *   - Each declaration cites the reference interface (file:line inside shinyoungkang1/mxfp4-int8-m5) it replaces.
 */
#ifndef SCMX_H_
#define SCMX_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SCMX_OK 0
#define SCMX_EINVAL (-1)   /* bad shape / argument */
#define SCMX_EFORMAT (-2)  /* unsupported weight format */
#define SCMX_ECUDA (-3)    /* CUDA runtime / driver error (launch failure, tensor-map encode failure) */
#define SCMX_EDEVICE (-4)  /* a bounded device-side wait ran out; the kernel returned early and set its status word */
#define SCMX_ELIMIT (-5)   /* size beyond a documented fixed limit */

/* Weight format: q[n,k] = +-code_mag[idx] * mult[bcode[n, k / block]]  (e2e/sc_format.py:26-41, `Format`). */
typedef struct scmx_format {
    int32_t block;        /* weights per block code along K; multiple of 8 */
    int32_t bc_bits;      /* bits per block code: 1, 2, 4 or 8 */
    int32_t n_mult;       /* entries used in mult[] (<= 2^bc_bits, <= 16) */
    int32_t code_mag[8];  /* magnitude of element index 0..7 */
    int32_t mult[16];     /* integer block multipliers; max(code_mag) * max(mult) <= 127 */
} scmx_format;

const char* scmx_last_error_string(void);
int scmx_abi_version(void);

/* ---- quantize / pack -------------------------------------------------------------------------------------- */

/* SC-MXFP4 quantizer + packer of an [N,K] matrix (K % 128 == 0) in float64 arithmetic.
 * Replaces sc_format.quantize (e2e/sc_format.py:105-111) = make_testcase.pack (sim/make_testcase.py:26-44) over
 * mx_int8.block_exponents(rule="search") / constrain_spread / dequant_mx / embed_int8 (sim/mx_int8.py:39-109).
 * w_dtype: 0 = float32, 1 = float64, 2 = bfloat16.  Outputs: codes u32 [N*K/8], bcodes u8 [N, K/128],
 * wscale f32 [N] = 2^(E_lo-1); optional qw int8 [N,K] and row_exp int32 [N] = E_lo (may be NULL). */
int scmx_quantize_sc_mxfp4(const void* w, int w_dtype, int64_t N, int64_t K, uint32_t* codes, uint8_t* bcodes,
                           float* wscale, int8_t* qw, int32_t* row_exp, void* stream);

/* Integer-exact format family quantizer in float32 arithmetic (row base search x per-block multiplier search).
 * Replaces formats.quantize (sim/formats.py:64-107) + pack_format.pack_parts (e2e/pack_format.py:53-76).
 * w float32 [N,K]; K/block <= 128 blocks per row and a multiple of 8.  Outputs as above; wscale = row base. */
int scmx_quantize_family(const float* w, int64_t N, int64_t K, const scmx_format* fmt, int base_grid,
                         uint32_t* codes, uint8_t* bcodes, float* wscale, int8_t* qw, void* stream);

/* Packed codes -> INT8 operand [N,K].  Replaces sc_kernels.unpack_i8 (e2e/sc_kernels.py:34-50,480-483). */
int scmx_unpack_i8(const uint32_t* codes, const uint8_t* bcodes, int64_t N, int64_t K, const scmx_format* fmt,
                   int8_t* wq, void* stream);

/* ---- activation row kernels --------------------------------------------------------------------------------- */

/* Per-token symmetric INT8: s = amax/127, q = clamp(rint(x * (1/s))), rows [M, Mp) zeroed.
 * Replaces sc_kernels.act_quant (e2e/sc_kernels.py:200-229,554-563).  x bf16 [M,K], K % 8 == 0. */
int scmx_act_quant(const uint16_t* x, int64_t M, int64_t K, int64_t Mp, int8_t* xq, float* xs, void* stream);

/* RMSNorm (weight nw bf16 [K]) then per-token INT8; xn (bf16 [Mp,K], may be NULL) receives the normalized rows.
 * Replaces sc_kernels.rmsnorm_quant / rmsnorm_quant_n (e2e/sc_kernels.py:123-174,527-533,619-626). */
int scmx_rmsnorm_quant(const uint16_t* x, const uint16_t* nw, float eps, int64_t M, int64_t K, int64_t Mp,
                       int8_t* xq, float* xs, uint16_t* xn, void* stream);

/* act_quant / rmsnorm_quant on rows stored as `nseg` column segments: element (m, s*w + j), w = K/nseg, lives at
 * x[s*seg_stride + m*w + j] (each segment a row-major [M, w] matrix, `seg_stride` elements apart) — the layout an
 * all-gather of column-sharded GEMM outputs leaves behind, consumed without a transposing copy.  The reference is
 * single-device and has no counterpart; the arithmetic is that of e2e/sc_kernels.py:200-229 / :123-174.  K <= 8192. */
int scmx_act_quant_seg(const uint16_t* x, int64_t M, int64_t K, int64_t Mp, int nseg, int64_t seg_stride, int8_t* xq,
                       float* xs, void* stream);
int scmx_rmsnorm_quant_seg(const uint16_t* x, const uint16_t* nw, float eps, int64_t M, int64_t K, int64_t Mp, int nseg,
                           int64_t seg_stride, int8_t* xq, float* xs, uint16_t* xn, void* stream);

/* h = res + T(acc * xscale[m] * wscale[n]) from INT32 accumulators [Mp,N].
 * Replaces sc_kernels.res_epilogue (e2e/sc_kernels.py:191-197,547-551). */
int scmx_res_epilogue(const int32_t* acc, const float* xscale, const float* wscale, const uint16_t* res, int64_t Mp,
                      int64_t N, uint16_t* h, void* stream);

/* SwiGLU of the bf16-rounded gate | up halves of INT32 accumulators [Mp, 2F], then per-token INT8 -> [Mp,F].
 * Replaces sc_kernels.swiglu_quant (e2e/sc_kernels.py:279-315,585-594). */
int scmx_swiglu_quant(const int32_t* acc, const float* xscale, const float* wscale, int64_t Mp, int64_t F,
                      int8_t* xq, float* xs, void* stream);

/* Elementwise sc_swiglu(g, u) on bf16 arrays of n elements (e2e/sc_kernels.py:319-328); used by the exhaustive
 * gate-value check the reference runs in e2e/test_sc_kernels.py:80-93. */
int scmx_swiglu(const uint16_t* g, const uint16_t* u, int64_t n, uint16_t* out, void* stream);

/* Rotated-input quantization: every 32-wide block of a row times a +-1 sign vector (signs f32 [K]) and the 32-point
 * Hadamard transform (float32 butterflies in the reference's order), scaled by 1/sqrt(32), rounded to bf16; then per-token
 * INT8 as scmx_act_quant.  Rows M..Mp-1 come out as zero codes with scale 0.  Replaces sc_kernels.rot_quant
 * (e2e/sc_kernels.py:234-275,572-582), the input side of weights packed in the rotated basis.  K % 32 == 0, K <= 8192. */
int scmx_rot_quant(const uint16_t* x, const float* signs, int64_t M, int64_t K, int64_t Mp, int8_t* xq, float* xs,
                   void* stream);

/* q/k/v epilogue between the fused q|k|v projection and attention.  src is the bf16 GEMM output y [L, (hq+2hk)d]
 * (src_is_acc = 0) or its int32 accumulators with xscale [L] and wscale [(hq+2hk)d] (src_is_acc != 0).  q and k get
 * T(w * T(x * inv)): per head over d values with qn / kn bf16 [d] (full = 0), or over the whole hq*d-wide q and hk*d-wide
 * k with qn bf16 [hq*d], kn bf16 [hk*d] (full != 0); v is copied.  Outputs are head-major: q[(h*q_head_stride + row)*d],
 * k and v at [(h*kv_head_stride + kv_row0 + row)*d], so k / v can be the rows of a cache of kv_head_stride positions.
 * inv_freq f32 [d/2] non-null: rotary embedding (half-split pairs i, i + d/2) at position pos0 + row applied to the
 * normalized q and k; rope_table (optional) f32 [rope_rows, d] holds cos (d/2 values) then sin (d/2) of
 * position * inv_freq per position, (float)cos((double)(float)(pos * inv_freq)): used instead of evaluating them
 * for positions < rope_rows.  pos_dev non-null: one device int32 added to pos0 and kv_row0 (rows beyond the cache are dropped).
 * Replaces qkv_epilogue_headnorm, qkv_headnorm_y, qkv_fullnorm_y (e2e/sc_kernels.py:333-423,597-637); the rotary step
 * and cache append replace the MLX calls of e2e/fused_qwen3.py:197-203.  d a power of two, row <= 48 KB as float. */
int scmx_qkv_norm(const void* src, int src_is_acc, const float* xscale, const float* wscale, const uint16_t* qn,
                  const uint16_t* kn, float eps, int64_t L, int hq, int hk, int d, int full, const float* inv_freq,
                  const float* rope_table, int64_t rope_rows, int64_t pos0, const int32_t* pos_dev, uint16_t* q, int64_t q_head_stride, uint16_t* k, uint16_t* v,
                  int64_t kv_head_stride, int64_t kv_row0, void* stream);

/* Batch-1 decode attention: out[h] = softmax(scale * q[h] K^T) V over the first T positions of a KV cache
 * (k_cache, v_cache bf16 [hk, capacity, d]; q bf16 [hq, d]; out bf16 [hq * d]).  T = pos_dev[0] + 1 when pos_dev is
 * non-null (a position counter kept on the device, so the call can be replayed from a CUDA graph while the sequence
 * grows), else n_pos.  The positions are split over nsplit CTAs per key/value head; partials f32 [hq, nsplit, d + 2]
 * and counters int32 [hk] (zero before the first call, left zero) are caller-provided scratch.
 * No counterpart in the reference, which calls MLX's scaled_dot_product_attention here (e2e/decode.py:103); outside
 * the W4A8 arithmetic: float32 online softmax, bf16 output.  d in {64, 128}, hq / hk in {1, 2, 4}. */
int scmx_attn_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, int64_t capacity,
                     const int32_t* pos_dev, int64_t n_pos, float scale, int hq, int hk, int d, int nsplit,
                     float* partials, int32_t* counters, uint16_t* out, void* stream);

/* ---- dense prefill GEMM (tcgen05 kind::i8) -------------------------------------------------------------------- */

/* out = epilogue(xq [M,K] . wq [N,K]^T).  epi 0: int32 [M,N] (mm_i8_i32, e2e/sc_kernels.py:53-71,486-495);
 * epi 1: bf16 T((float(acc)*xscale[m])*wscale[n]); epi 2: bf16 T(res + T(...)); epi 3: SwiGLU of interleaved
 * gate/up column groups -> bf16 [M, N/2]  (mm_epi, e2e/sc_kernels.py:79-115,498-508).
 * K % 16 == 0, N % 32 == 0, all row pitches 16-byte aligned.  status: device int32[4], zero-filled by the caller
 * once; non-zero afterwards means a bounded wait inside the kernel ran out (results invalid). */
int scmx_mm_i8(const int8_t* xq, const int8_t* wq, int64_t M, int64_t N, int64_t K, int epi, const float* xscale,
               const float* wscale, const uint16_t* res, void* out, int32_t* status, void* stream);

/* Process-wide tuning hint for the N tile of the GEMM kernels: 0 = automatic, 128 or 256.  Counterpart of the
 * module-level tile constants TM, TN, NSG, GROUP_M (e2e/sc_kernels.py:25) and the `tile=` arguments. */
int scmx_set_gemm_tile(int bn);
/* Process-wide switch (default on): dense GEMMs with M > 128 and N >= 256 run on pairs of CTAs that share a 256 x 256 tile
 * (tcgen05 cta_group::2); off = every CTA computes 128 x 256 tiles of its own.  Same results.  scmx_set_gemm_tile with a
 * non-zero value also selects the single-CTA kernel.  No counterpart in the reference. */
int scmx_set_gemm_pair(int enable);

/* Process-wide switches with no counterpart in the reference: programmatic dependent launch for the kernels of the chains
 * (default on) and the streaming (bulk-copy, persistent) form of the dense GEMV: mode 0 = never, 1 = for matrices of
 * 16 MB of packed codes and more (default), 2 = whenever the shape allows it; other values are refused.  For A/B
 * measurements and for tests of the streaming kernel on small shapes. */
int scmx_set_pdl(int enable);
int scmx_set_gemv_stream(int mode);

/* Limit, in nanoseconds, of every bounded device-side wait of kernels launched afterwards (mbarrier waits of the GEMM
 * and the streaming GEMV, the flag wait of scmx_peer_barrier); default 2 s, accepted range 1 us .. 60 s.  A wait that
 * runs out stores a code in the kernel's status word (1..5 GEMM roles, 11 / 12 streaming GEMV, 20 peer barrier) and the
 * kernel returns early.  Process-wide; no counterpart in the reference (failure detection, outside its scope). */
int scmx_set_wait_limit_ns(unsigned long long ns);
/* Registers, for the current device, the int32[4] status word used by kernels whose entry point takes no status
 * argument (scmx_gemv's streaming kernel).  NULL (the default) = such kernels give up silently. */
int scmx_set_status_word(int32_t* status);

/* ---- grouped MoE GEMM ------------------------------------------------------------------------------------------- */

/* Counting sort of M*topk assignments by expert with segment offsets and M-tile starts.
 * Replaces sc_moe.route_sort (e2e/sc_moe.py:114-155).  inds int32 [M,topk]; outputs pos int32 [M*topk],
 * tok int32 [M*topk + tm], esorted int32 [M*topk], off int32 [E+1], tstart int32 [E+1].  E <= 1024. */
int scmx_route_sort(const int32_t* inds, int64_t M, int topk, int E, int tm, int32_t* pos, int32_t* tok,
                    int32_t* esorted, int32_t* off, int32_t* tstart, void* stream);

/* Router: softmax over E logits per token then the topk largest (ties to the lower expert id), scores not
 * renormalised.  Replaces the MLX ops of e2e/fused_olmoe.py:216-220.  logits f32 [M,E]; inds int32 [M,topk];
 * scores bf16 [M,topk]; scores_f32 (may be NULL) f32 [M,topk]. */
int scmx_router_topk(const float* logits, int64_t M, int E, int topk, int32_t* inds, uint16_t* scores,
                     float* scores_f32, void* stream);

/* Row gather: dst_q[p] = xq[tok[p]] for p < rows_q, dst_s[p] = xs[tok[p]] for p < rows_s
 * (the `xq[tok_p], xs[tok_p[:R]]` of e2e/fused_olmoe.py:230). */
int scmx_gather_rows(const int8_t* xq, const float* xs, const int32_t* tok, int64_t rows_q, int64_t rows_s, int64_t K,
                     int8_t* dst_q, float* dst_s, void* stream);

/* Grouped GEMM over expert segments from pre-unpacked INT8 weights wq [E*N, K]; rows [off[e], off[e+1]) of xq use
 * expert e.  Replaces sc_moe.moe_mm_i8 (e2e/sc_moe.py:97-107,188-200).  epi 0/1/3 as scmx_mm_i8 with
 * wscale f32 [E,N].  tm must be 128 (the M tile of the kernel; off/tstart must come from route_sort with that tm). */
int scmx_moe_mm_i8(const int8_t* xq, int64_t R, const int8_t* wq, const float* wscale, const int32_t* off,
                   const int32_t* tstart, int E, int64_t N, int64_t K, int epi, const float* xscale, void* out,
                   int tm, int32_t* status, void* stream);

/* Grouped GEMM straight from packed weights: codes u32 [E, N*K/8], bcodes u8 [E, N, K*bc_bits/(8*block)].
 * Replaces sc_moe.moe_mm (e2e/sc_moe.py:19-92,169-185).  Expert weights are decoded to INT8 in groups of
 * `experts_per_pass` experts into `scratch` (caller-provided, >= 2 * experts_per_pass * N * K bytes, two rotating
 * halves that stay L2-resident) and consumed by the tcgen05 grouped kernel. */
int scmx_moe_mm(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                const int32_t* off, const int32_t* tstart, int E, int64_t N, int64_t K, const scmx_format* fmt, int epi,
                const float* xscale, void* out, int tm, int experts_per_pass, int8_t* scratch, int64_t scratch_bytes,
                int32_t* status, void* stream);

/* The GEMMs straight from packed weights, single pass: the 4-bit tiles are expanded to INT8 in shared memory inside the K
 * loop of the tensor-core kernel (CTA pairs; four unpack warps per CTA), so decoded weights never reach global memory and
 * no scratch is needed.  scmx_mm_w4 = scmx_mm_i8 on unpack_i8's output, the single-pass W4A8 linear of the reference
 * (kernels/w4a8.metal:78-155, e2e/w4a8_mlx.py:88-135); scmx_moe_mm_w4 = sc_moe.moe_mm with its in-kernel unpack
 * (e2e/sc_moe.py:19-92,169-185).  Same results as the two-kernel forms, bit for bit.  Format rule: K % 128 == 0 and the
 * block codes of 128 weights form one field of 8, 16 or 32 bits (block 32 / 2-bit codes, block 16 / 2- or 4-bit codes, ...;
 * scmx_w4_supported returns 1 when a format and K qualify).  Grouped form: E <= 512, rows [off[e], off[e+1]) use expert e;
 * no tile table is needed (the kernel derives its own 256-row tiles from off).  status codes as scmx_mm_i8, plus 6 =
 * an unpack warp waited for a packed tile. */
int scmx_w4_supported(const scmx_format* fmt, int64_t K);
int scmx_mm_w4(const int8_t* xq, const uint32_t* codes, const uint8_t* bcodes, int64_t M, int64_t N, int64_t K,
               const scmx_format* fmt, int epi, const float* xscale, const float* wscale, const uint16_t* res, void* out,
               int32_t* status, void* stream);
int scmx_moe_mm_w4(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                   const int32_t* off, int E, int64_t N, int64_t K, const scmx_format* fmt, int epi, const float* xscale,
                   void* out, int32_t* status, void* stream);

/* scmx_moe_mm_w4 with the row-mapped epilogue of scmx_moe_mm_i8_ret (EPI 1; output row r stored at row ret_row[r] of
 * out_peers[ret_rank[r]]): the down GEMM of the expert-parallel block when the weights are read packed. */
int scmx_moe_mm_w4_ret(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                       const int32_t* off, int E, int64_t N, int64_t K, const scmx_format* fmt, const float* xscale,
                       const int32_t* ret_rank, const int32_t* ret_row, int world, void* const* out_peers, int32_t* status,
                       void* stream);

/* scmx_moe_mm without a scratch argument; it has no counterpart in the reference (whose arrays are allocated by MLX).
 * For hosts that cannot hand the library device memory at call time: a serving process that gave all of HBM to its own
 * pool at start-up (a cudaMalloc there would fail, or stall the device mid-request), or a foreign-language runtime bound
 * to this C ABI that owns no device allocator.  The decoded-INT8 staging area is a fixed 16 MiB array inside the library
 * (two 8 MiB halves), held by every GPU that loads the library until the process exits.  The call allocates nothing.
 * Limit: one decoded expert matrix must fit one half, N * K <= 8 MiB (8388608); larger shapes return SCMX_ELIMIT.
 * The first call on a device looks up the array's device address (and, for epi 3, builds the SiLU table and
 * synchronises the stream once): make that first call before any stream capture (during capture it is refused with
 * SCMX_EINVAL).  The array comes into being when the library's code is first loaded on a device, so a host that
 * reserves all remaining device memory for itself should make one warm-up call per device before doing so.  All calls share the one array:
 * every byte read from it is rewritten by the same call first, so contents left by an earlier call are never used,
 * but two calls whose kernels overlap on the GPU (different streams, or different threads on the same device) race. */
int scmx_moe_mm_static(const int8_t* xq, int64_t R, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
                       const int32_t* off, const int32_t* tstart, int E, int64_t N, int64_t K, const scmx_format* fmt,
                       int epi, const float* xscale, void* out, int tm, int32_t* status, void* stream);

/* ---- expert-parallel exchange over peer memory (multi-GPU; the reference is single-device and has no counterpart) ----
 * `*_peers` are HOST arrays of `world` device pointers: entry r is the buffer of that name on rank r's GPU, mapped into
 * this process (CUDA IPC), entry `rank` the local one.  Buffers per GPU: rx_q int8 [world, cap, K], rx_s f32 [world, cap],
 * rx_meta int32 [world, E/world + 1], y_back bf16 [cap, D], flags int32 [world] (zeroed once), epoch int32 [1] (zeroed once).
 * cap = the most rows one rank can send (tokens_per_rank * topk).  world <= 8, E/world <= 128. */

/* Stores every sorted assignment row (xq[tok[p]], xs[tok[p]]) into the owner rank's rx_q / rx_s at [rank][p - off[first
 * expert of the owner]], and the per-expert counts plus that base row into the owner's rx_meta[rank]. */
int scmx_ep_dispatch(const int8_t* xq, const float* xs, const int32_t* tok, const int32_t* esorted, const int32_t* off,
                     int64_t R, int64_t K, int E, int world, int rank, int64_t cap, const void* const* rx_q_peers,
                     const void* const* rx_s_peers, const void* const* rx_meta_peers, void* stream);
/* All-gather by stores: writes `bytes` from src at dst_offset_bytes into every rank's buffer dst_peers[r] (own included).
 * Follow with scmx_peer_barrier before reading the gathered buffer.  16-byte granularity. */
int scmx_peer_put(const void* src, int64_t bytes, int64_t dst_offset_bytes, const void* const* dst_peers, int world, void* stream);
/* All ranks signal each other and wait for everyone (bounded to 2 s, then status[0] = 20). */
int scmx_peer_barrier(const void* const* flag_peers, int rank, int world, int32_t* epoch, int32_t* status, void* stream);
/* From rx_meta: expert segments off2 / tstart2 [El+1], the regrouping gather list tok2 [r_cap + tm] (rows of rx_q in
 * expert-major order), the return address (ret_rank, ret_row) of every regrouped row, and n_rows[0] = rows received. */
int scmx_ep_plan(const int32_t* rx_meta, int world, int El, int64_t cap, int tm, int64_t r_cap, int32_t* off2,
                 int32_t* tstart2, int32_t* tok2, int32_t* ret_rank, int32_t* ret_row, int32_t* n_rows, void* stream);
/* Stores expert output row p (bf16 [D]) into rank ret_rank[p]'s y_back at row ret_row[p], for p < n_rows[0]. */
int scmx_ep_return(const uint16_t* y, const int32_t* ret_rank, const int32_t* ret_row, const int32_t* n_rows, int64_t r_cap,
                   int64_t D, int world, const void* const* y_back_peers, void* stream);
/* scmx_mm_i8 whose epilogue IS the all-gather of tensor parallelism: every output line is stored at the same row and column
 * of out_peers[0 .. world) (HOST array of device pointers: each GPU's copy of the output segment of THIS rank, this GPU's own
 * included; peer buffers are peer-mapped memory), straight from the staged epilogue in full 128-byte lines.  Follow with
 * scmx_peer_barrier before any rank reads.  epi 1, 2 or 3; M > 128 and N >= 256 (the CTA-pair kernel).  Replaces
 * scmx_mm_i8 + scmx_peer_put.  No counterpart in the single-device reference. */
int scmx_mm_i8_bcast(const int8_t* xq, const int8_t* wq, int64_t M, int64_t N, int64_t K, int epi, const float* xscale,
                     const float* wscale, const uint16_t* res, void* const* out_peers, int world, int32_t* status, void* stream);
/* scmx_moe_mm_i8 with EPI 1 whose epilogue IS the return exchange of expert parallelism: bf16 output row r of the grouped
 * GEMM is stored at row ret_row[r] of out_peers[ret_rank[r]] (bf16 [*, N] buffers of the `world` GPUs, this GPU's own
 * included; peer buffers are device pointers of peer-mapped memory), straight from the TMEM accumulators, instead of being
 * written locally and moved by scmx_ep_return afterwards.  ret_rank / ret_row as produced by scmx_ep_plan; rows outside the
 * expert segments (off) are not stored.  Follow with scmx_peer_barrier before the peers read.  No counterpart in the
 * single-device reference. */
int scmx_moe_mm_i8_ret(const int8_t* xq, int64_t R, const int8_t* wq, const float* wscale, const int32_t* off,
                       const int32_t* tstart, int E, int64_t N, int64_t K, const float* xscale, const int32_t* ret_rank,
                       const int32_t* ret_row, int world, void* const* out_peers, int tm, int32_t* status, void* stream);
/* scmx_moe_combine whose expert rows are READ from the GPUs that computed them (expert parallelism, "pull" form): y_peers[d]
 * is rank d's output buffer bf16 [world * cap, K] ordered by receive slot (source rank * cap + position among the rows that
 * source sent), as written by scmx_moe_mm_i8_ret with ret_row = the gather list of scmx_ep_plan.  Sorted position p of this
 * rank (pos, esorted, off from scmx_route_sort over the GLOBAL expert ids) lives at y_peers[esorted[p] / El][rank * cap +
 * p - off[(esorted[p] / El) * El]].  Same arithmetic as scmx_moe_combine; replaces scmx_ep_return + the barrier-separated
 * local combine by one kernel that loads over peer memory.  Run scmx_peer_barrier first.  No counterpart in the reference. */
int scmx_moe_combine_pull(const void* const* y_peers, int world, int rank, int El, int64_t cap, const int32_t* esorted,
                          const int32_t* off, const int32_t* pos, const uint16_t* scores, const uint16_t* res,
                          const uint16_t* nw, float eps, int64_t M, int64_t Mp, int64_t K, int topk, int quant, uint16_t* h,
                          int8_t* xq, float* xs, void* stream);
/* gather_rows / act_quant over a device-side row count: rows >= n_rows[0] + pad are skipped, the pad rows after
 * n_rows[0] are zero-filled. */
int scmx_gather_rows_dyn(const int8_t* xq, const float* xs, const int32_t* tok, const int32_t* n_rows, int64_t r_cap, int pad,
                         int64_t K, int8_t* dst_q, float* dst_s, void* stream);
int scmx_act_quant_dyn(const uint16_t* x, const int32_t* n_rows, int64_t r_cap, int pad, int64_t K, int8_t* xq, float* xs,
                       void* stream);
int scmx_enable_peer_access(int peer_device);

/* Weighted sequential-bf16 sum of the topk expert rows + residual (+ next RMSNorm + INT8 when quant != 0).
 * Replaces fused_olmoe.moe_combine (e2e/fused_olmoe.py:45-97).  y bf16 [R,K], pos int32 [M*topk], scores bf16
 * [M,topk], res bf16 [Mp,K] -> h bf16 [Mp,K], xq int8 [Mp,K], xs f32 [Mp]. */
int scmx_moe_combine(const uint16_t* y, const int32_t* pos, const uint16_t* scores, const uint16_t* res,
                     const uint16_t* nw, float eps, int64_t M, int64_t Mp, int64_t K, int topk, int quant,
                     uint16_t* h, int8_t* xq, float* xs, void* stream);

/* ---- batch-1 decode GEMV ------------------------------------------------------------------------------------------ */

/* y[slot, n] = epilogue(xscale * wscale[n] * sum_k xq[k] q[n,k]) reading the packed codes directly.
 * Replaces sc_decode.gemv (e2e/sc_decode.py:19-183,208-238) with pro = 0.  n_slots = 1 and eidx = NULL: dense.
 * MoE: slot j uses expert eidx[j] (or `shared` for slot n_routed when shared >= 0) and input row j * xstride.
 * epi 1/2/3 as scmx_mm_i8 (epi 2 reads res bf16 [N]); epi 0 writes the exact int32 totals.
 * K % 128 == 0, N % 4 == 0.  pdl != 0 launches with programmatic stream serialization so the weight loads of
 * this call overlap the tail of the previous kernel on the stream. */
int scmx_gemv(const int8_t* xq, const float* xscale, const uint32_t* codes, const uint8_t* bcodes, const float* wscale,
              int64_t N, int64_t K, const scmx_format* fmt, int epi, const uint16_t* res, const int32_t* eidx,
              int n_routed, int shared, int xstride, void* out, int pdl, void* stream);

/* Many independent dense GEMVs in one persistent launch.  A job is one y = epilogue(W x) as in scmx_gemv (no expert
 * gather, no prologue); all jobs share the weight format.  The kernel streams the packed weights of all jobs through one
 * shared-memory ring without pausing at matrix boundaries, so a list of small GEMVs runs at streaming bandwidth instead of
 * paying a launch and a pipeline fill each.  Counterpart of issuing sc_decode.gemv once per weight set
 * (e2e/sc_decode.py:208-238), batched the way the reference times it: a list of calls evaluated as one graph
 * (e2e/tune_07.py:19-28).  Inputs of every job must be complete when the launch starts (jobs cannot feed each other).
 * Limits: K % 128 == 0, K <= 8192, N % 4 == 0, K*bc_bits/(8*block) % 4 == 0, block 8, 16 or a multiple of 32, at most 512
 * jobs; codes, bcodes, wscale and xq 16-byte aligned. */
typedef struct scmx_gemv_job {
    const uint32_t* codes;   /* u32 [N*K/8] */
    const uint8_t* bcodes;   /* u8 [N, K*bc_bits/(8*block)] */
    const float* wscale;     /* f32 [N] */
    const int8_t* xq;        /* int8 [K] */
    const float* xscale;     /* f32 [1] (unused for epi 0) */
    const uint16_t* res;     /* bf16 [N], epi 2 only */
    void* out;               /* epi 0: int32 [N]; 1, 2: bf16 [N]; 3: bf16 [N/2] */
    int32_t N, K, epi;
    int32_t plan[15];        /* filled by scmx_gemv_multi_plan; opaque */
} scmx_gemv_job;
/* Validates a HOST array of n jobs and fills their plan fields (tile shapes and the position of each job in the launch). */
int scmx_gemv_multi_plan(scmx_gemv_job* jobs_host, int n, const scmx_format* fmt);
/* Launches the planned list.  jobs_host: the planned host array; jobs_dev: a device copy of the same n records made by the
 * caller after planning (ignored for n = 1).  status as in scmx_mm_i8 (codes 11 / 12). */
int scmx_gemv_multi(const scmx_gemv_job* jobs_host, const scmx_gemv_job* jobs_dev, int n, const scmx_format* fmt,
                    int32_t* status, int pdl, void* stream);

/* scmx_gemv on a bf16 input row (or rows, xstride = 1) quantized inside the kernel: pro = 1 per-token INT8
 * (scmx_act_quant's arithmetic), pro = 2 RMSNorm with weights nw bf16 [K] and eps first (scmx_rmsnorm_quant's).
 * Every CTA computes the INT8 row in shared memory after its weight loads are in flight; results are bit-identical to
 * the row kernel followed by scmx_gemv.  Replaces the PRO 1 / PRO 2 prologues of sc_decode.gemv
 * (e2e/sc_decode.py:50-65).  K <= 8192, epi in 1..3; always the register kernel (no streaming variant). */
int scmx_gemv_pro(const uint16_t* x, int pro, const uint16_t* nw, float eps, const uint32_t* codes, const uint8_t* bcodes,
                  const float* wscale, int64_t N, int64_t K, const scmx_format* fmt, int epi, const uint16_t* res,
                  const int32_t* eidx, int n_routed, int shared, int xstride, void* out, int pdl, void* stream);

/* ---- one decode step of a dense stack as a persistent kernel ------------------------------------------------------------- */

/* Weights of one decoder layer for scmx_decode_step_dense: [0] q|k|v rows concatenated, [1] o, [2] gate|up with rows
 * interleaved for the SwiGLU epilogue, [3] down; SC-MXFP4 in the default format (block 32, shifts).  k_cache / v_cache:
 * bf16 [hk, capacity, d]. */
typedef struct scmx_decode_layer {
    const uint32_t* codes[4];
    const uint8_t* bcodes[4];
    const float* wscale[4];
    const uint16_t* ln_in;     /* input RMSNorm weights, bf16 [D] */
    const uint16_t* ln_post;   /* post-attention RMSNorm weights, bf16 [D] */
    const uint16_t* q_norm;    /* bf16 [d] */
    const uint16_t* k_norm;    /* bf16 [d] */
    uint16_t* k_cache;
    uint16_t* v_cache;
} scmx_decode_layer;

/* All layers of one batch-1 decode step in one cooperative launch: h bf16 [D] (in: the token's embedding, out: the residual
 * stream after the last layer) goes through n_layers of RMSNorm + INT8 -> q|k|v GEMV -> q/k head RMSNorm + rotary embedding
 * + cache append at row pos_dev[0] -> attention over pos_dev[0] + 1 positions -> o GEMV + residual -> RMSNorm + INT8 ->
 * gate|up GEMV with SwiGLU -> INT8 -> down GEMV + residual, the chain of e2e/decode.py:58-110, with grid-wide barriers
 * between the steps instead of kernel boundaries.  Same bits as scmx_rmsnorm_quant / scmx_gemv / scmx_qkv_norm /
 * scmx_attn_decode (with the same nsplit) / scmx_act_quant called in that order.
 * layers: device array; y bf16 [(hq + 2 hk) d], act bf16 [F], o bf16 [hq d], partials f32 [hq, nsplit, d + 2], barrier
 * uint32 [2] are scratch; counters int32 [hk] is scratch too (zeroed by every call on its stream); status int32 [1] receives 100 + k if barrier k timed out (0.5 s), after which the step's outputs are invalid.
 * Limits: d = 128; D, F and hq*d multiples of 1024 up to 6144; hq/hk in {1, 2, 4}; hk * nsplit <= number of SMs.
 * Not to be run concurrently with other work on the same device: the launch needs every SM. */
int scmx_decode_step_dense(const scmx_decode_layer* layers, int n_layers, int D, int F, int hq, int hk, int d, float eps,
                           float scale, const float* inv_freq, const float* rope_table, int64_t rope_rows, int64_t capacity,
                           const int32_t* pos_dev, uint16_t* h, uint16_t* y, uint16_t* act, uint16_t* o, float* partials,
                           int nsplit, int32_t* counters, uint32_t* barrier, int32_t* status, void* stream);
/* Diagnostic: while device_buf is set, CTA 0 of scmx_decode_step_dense stores its SM cycle counter in device_buf[0 .. n)
 * at every barrier entry and exit and, in the attention phase, after the q/k/v preparation and after the split's positions,
 * layer after layer; with
 * n_and_barrier = n | (b << 16), b > 0, every CTA also stores the global nanosecond timer at its arrival at barrier b
 * (1-based) in device_buf[n + CTA index].  device_buf: uint64 [n + number of SMs].  0 switches it off.  Process-wide; no
 * counterpart in the reference. */
int scmx_set_decode_trace(unsigned long long* device_buf, int n_and_barrier);

#ifdef __cplusplus
}
#endif
#endif /* SCMX_H_ */
