/*
 * linghe_b200 -- C ABI of the sm_100a fused norm / SwiGLU + FP8 e4m3 blockwise
 * quantisation kernels.
 *
 * This is the drop-in boundary: plain pointers and sizes, no framework types.  Each
 * entry point replaces one host wrapper of the upstream Python/Triton library
 * (inclusionAI/linghe, paths below are inside that project) and keeps its tensor and
 * scale layouts byte for byte.
 *
 * Conventions
 *   - All pointers are device pointers on the current CUDA device unless said
 *     otherwise; `stream` is a cudaStream_t (NULL = legacy default stream).
 *   - Work is enqueued asynchronously; no entry point synchronises or allocates,
 *     except where stated.  Scratch memory, when needed, is passed in by the caller.
 *   - Return value: 0 = enqueued; LH_ERR_ARG (<0) = rejected arguments (nothing was
 *     launched); >0 = a cudaError_t from the launch.  lh_last_error() returns a
 *     thread-local message for the last non-zero return.
 *   - `dtype`: element type of the floating-point inputs (LH_BF16 / LH_F16 / LH_F32).
 *     Every entry point accepts all three except lh_rmsnorm_gemm_blockquant_fwd (LH_BF16);
 *     gamma and the incoming gradient have the type of x, bf16 outputs that of the input.
 *   - fp8 outputs are e4m3fn codes (1 byte each); scales are float32 dequantisation
 *     multipliers: scale = max(amax/448, 1e-30), optionally rounded up to a power of 2.
 *   - `output_mode`: 0 = row-wise (1x128) outputs only, 1 = column-wise (128x1,
 *     transposed) outputs only, 2 = both.  Pointers of outputs a mode does not write
 *     may be NULL.
 *   - Layouts (nb = n/128, i row, j column, b = j/128, I = i/128):
 *       q  [M,n]            offset i*n + j
 *       s  [nb,M]           offset b*M + i            (row scales, transposed)
 *       qT [n,M]            offset j*M + i
 *       sT [ceil(M/128),n]  offset I*n + j
 *     Per-expert (batched) entry points pack, for expert e with c_e rows starting at
 *     row S_e and B_e = sum_{e'<e} ceil(c_e'/128):
 *       q  offset (S_e+t)*n + j
 *       s  offset S_e*nb + b*c_e + t
 *       qT offset S_e*n + j*c_e + t
 *       sT offset (B_e + t/128)*n + j
 */
#ifndef LINGHE_B200_H_
#define LINGHE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LH_VERSION 100

#define LH_OK 0
#define LH_ERR_ARG (-1)

enum { LH_BF16 = 0, LH_F16 = 1, LH_F32 = 2, LH_U8 = 3 /* raw bytes: e4m3 codes */ };
enum { LH_I32 = 0, LH_I64 = 1 };

/* Library version (LH_VERSION of the build). */
int lh_version(void);

/* Message for the last non-zero return on this thread ("" if none). */
const char* lh_last_error(void);

/* 0 if `device` is an sm_100 GPU these kernels can run on, LH_ERR_ARG otherwise. */
int lh_device_check(int device);

/* Copies the device status word of the current device to *status (0 = no kernel ever
 * gave up on a bounded wait) and clears it.  Synchronises the device. */
int lh_device_status(int* status);

/* Self-test of the give-up path of the kernels' bounded waits.  Launches one warp that
 * waits `polls` polls (1..65536) on a barrier nobody arrives at, records the status code
 * of a timed-out tile wait (1) in the device status word and returns, as a production
 * kernel whose copy never landed would.  lh_device_status() then reports 1 once and 0
 * afterwards.  No counterpart in the reference (Triton kernels have no such waits).
 *
 * Every wait inside the kernels is bounded (about two seconds of SM clock).  A wait that
 * runs out does not abort the kernel: the kernel finishes with undefined outputs and the
 * status word set, and entry points keep returning 0 because they never synchronise.
 * Callers that want to detect this poll lh_device_status() at a point where they
 * synchronise anyway (end of a step). */
int lh_selftest_wait_timeout(int polls, void* stream);

/* Measurement switch: sets the named dispatch option and returns its previous value
 * (LH_ERR_ARG for an unknown key).  Process-wide; meant for A/B timing, not for production.
 *   "rmsnorm_both_single_pass"   mode 2 of lh_rmsnorm_blockquant_fwd: 0 = row kernel then column
 *                                kernel, 1 (default) = the single-pass kernel for n < 6144, where
 *                                it is ahead, 2 = the single-pass kernel at every width
 *   "rmsnorm_bwd_quant_single_pass"        lh_rmsnorm_bwd_blockquant: 1 = the single-pass cluster
 *                                kernel (x and dy read from HBM once), 0 (default) = two launches
 *   "rmsnorm_bwd_quant_two_role_min_n"   lh_rmsnorm_bwd_blockquant: rows at least this wide take
 *                                the streaming kernel with a second role per CTA that writes the
 *                                transposed copy tile by tile beside the walk (default: never)
 *   "second_launch_descends"     1 (default) = the second launch of a two-launch path walks the row
 *                                bands last to first, starting with what the first left in L2
 *   "band_cluster"               cluster size of the single-pass kernels: 0 = chosen per shape, else 1 / 2 / 4 / 8
 *   "rmsnorm_bwd_stream_min_n"   lh_rmsnorm_bwd: rows at least this wide take the streaming register kernel,
 *                                narrower ones the TMA ring (default 1536) */
int lh_tuning(const char* key, int value);

/* Scratch bytes needed by the entry point named `what` ("rmsnorm_bwd",
 * "batch_silu_bwd") for the given sizes; 0 if it needs none, <0 if unknown. */
int64_t lh_scratch_bytes(const char* what, int64_t rows, int64_t cols);

/* ---- pure quantisers (bit-exact against the PyTorch reference math) ------------ */

/* Dual-axis activation quantiser.
 * Replaces triton_blockwise_quant, linghe/quant/block.py:129.
 * x [M,N] contiguous, N % 128 == 0. */
int lh_blockwise_quant(const void* x, int dtype, int64_t M, int64_t N, void* q, float* s, void* qt,
                       float* st, int round_scale, int output_mode, void* stream);

/* Row-only 1x128 quantiser with untransposed scales s [M, N/128].
 * Replaces triton_group_quant, linghe/quant/group.py:40. */
int lh_group_quant(const void* x, int dtype, int64_t M, int64_t N, void* q, float* s, int round_scale,
                   void* stream);

/* 128x128 2-D block quantiser for weights, s [M/128, N/128], no scale floor in the
 * reference oracle but the kernel floors at 1e-30 like the upstream kernel.
 * Replaces triton_block_quant, linghe/quant/block.py:32.  M,N multiples of 128. */
int lh_block_quant(const void* x, int dtype, int64_t M, int64_t N, void* q, float* s, int round_scale,
                   void* stream);

/* Per-expert dual-axis quantiser with packed outputs.
 * Replaces triton_batch_blockwise_quant, linghe/quant/block.py:251.
 * counts: device array of E row counts (LH_I32 / LH_I64); R = total rows. */
int lh_batch_blockwise_quant(const void* x, int dtype, const void* counts, int counts_type, int E,
                             int64_t R, int64_t N, void* q, float* s, void* qt, float* st,
                             int round_scale, void* stream);

/* Gather rows by index into per-expert segments padded to multiples of 16 rows, and
 * quantise them on both axes (the step that feeds the routed experts).
 * Replaces triton_batch_block_pad_permute_with_indices, linghe/utils/gather.py:1049.
 * x [m,N]; counts [E] rows per expert (device); indices [M_out] source row of every
 * padded output position (entries of padding positions are ignored), M_out = sum of the
 * padded counts; probs optional [m,E] with prob_out [M_out] in probs_dtype (LH_F32 /
 * LH_BF16; padding positions get 0).  Outputs use the per-expert packed layouts with
 * c_e = padded count; padding rows are zero rows (scale floor 1e-30, codes 0). */
int lh_batch_block_pad_permute(const void* x, int dtype, const void* probs, int probs_dtype,
                               const void* indices, int indices_type, const void* counts, int counts_type,
                               int E, int64_t m, int64_t M_out, int64_t N, void* q, float* s, void* qt,
                               float* st, void* prob_out, int round_scale, void* stream);

/* ---- RMSNorm ------------------------------------------------------------------- */

/* y = (x * r) * gamma in the input dtype, r = rsqrt(mean(x^2) + eps) per row.
 * Replaces triton_rms_norm_forward, linghe/utils/norm.py:58.
 * reuse_rms != 0: read r from `rms` instead of computing (and do not write it). */
int lh_rmsnorm_fwd(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* y,
                   float* rms, int reuse_rms, void* stream);

/* RMSNorm + blockwise quantisation.
 * Replaces triton_rms_norm_and_block_quant_forward, linghe/utils/norm.py:343.
 * mode 0: writes q, s, rms.  mode 1: reads rms, writes qT, sT.  mode 2: writes all.
 * n % 128 == 0, except mode 1, which takes n % 32 == 0 as upstream does (linghe/utils/norm.py:416-419).
 * Mode 2 with bf16 inputs and n < 6144 is ONE kernel that reads x from HBM once (upstream runs
 * two kernels, linghe/utils/norm.py:464-500, and reads x twice); wider rows run a row kernel
 * followed by a column kernel, which is faster there. */
int lh_rmsnorm_blockquant_fwd(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps,
                              void* q, float* s, float* rms, void* qt, float* st, int round_scale,
                              int output_mode, void* stream);

/* RMSNorm + float32 router logits + row quantisation (the step beside the norm in the MoE block).
 * Replaces triton_rms_norm_fp32_gemm_block_quant_forward, linghe/utils/norm.py:688.
 * x [M,K] bf16, gamma [K] bf16, route_w [N,K] bf16; M, K, N multiples of 128, K <= 8192.
 * mode 0: writes y [M,K] bf16, rms [M], logits [M,N] f32 = y_f32 . route_w^T, q [M,K], s [K/128,M].
 * mode 1: reads rms, writes qT [K,M], sT [M/128,K] (y, logits, q, s untouched).
 * scratch: lh_scratch_bytes("rmsnorm_gemm", N, K) bytes (mode 0 only). */
int lh_rmsnorm_gemm_blockquant_fwd(const void* x, const void* gamma, const void* route_w, int dtype, int64_t M,
                                   int64_t K, int64_t N, float eps, void* y, float* rms, float* logits, void* q,
                                   float* s, void* qt, float* st, int round_scale, int output_mode, void* scratch,
                                   int64_t scratch_bytes, void* stream);

/* RMSNorm backward: dx (input dtype) and dgamma (float32 [n]).
 * Replaces triton_rms_norm_backward, linghe/utils/norm.py:144.
 * rms may be NULL (recomputed).  scratch: lh_scratch_bytes("rmsnorm_bwd", M, n) bytes. */
int lh_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                   int64_t n, float eps, void* dx, float* dgamma, void* scratch, int64_t scratch_bytes,
                   void* stream);

/* RMSNorm backward for callers that must not allocate device memory.
 * No counterpart in the reference (its wrapper always allocates a partial buffer with
 * torch.empty): this is lh_rmsnorm_bwd with the dgamma scratch built into the library.
 *
 * Who needs it: host code that sits outside the framework's caching allocator -- a plain
 * C/C++ integration of this ABI, or a training job that has already handed all free
 * device memory to its pool -- cannot get scratch for lh_rmsnorm_bwd: a raw cudaMalloc
 * may fail for lack of memory, and cudaMalloc / cudaFree stall the device besides.
 * Here the per-CTA partial sums go to a fixed device array of 148 x 8192 floats
 * (4 849 664 bytes) that every GPU holds from the moment it loads the library until the
 * process exits.  The call performs no cudaMalloc, cudaFree or any other allocation.
 *
 * Limits and rules:
 *   - n <= 8192 (and n % 128 == 0); larger n is rejected with LH_ERR_ARG.  M is unbounded.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) and caches it; make that first call with the device current
 *     and before starting any stream capture.
 *   - All calls on a device share the one array, which keeps whatever the last call left
 *     in it.  Nothing needs clearing (each call overwrites every partial row it later
 *     reads), but two calls whose kernels overlap on the GPU -- different streams, or
 *     different host threads on different streams -- race on it: serialise them.
 * Arguments as lh_rmsnorm_bwd without the scratch pair.  dx and dgamma agree with
 * lh_rmsnorm_bwd to within float32 summation order: for n < 1536 on a 148-SM device both
 * run the same kernel on the same grid and the results are bit-identical; for wider rows
 * lh_rmsnorm_bwd takes a different kernel, so the last bits of dgamma (and, through the
 * row sums, of a few dx values) may differ. */
int lh_rmsnorm_bwd_static(const void* dy, const void* x, const void* gamma, const float* rms, int dtype,
                          int64_t M, int64_t n, float eps, void* dx, float* dgamma, void* stream);

/* RMSNorm backward fused with the dual-axis quantisation of dy (the copies the
 * neighbouring linear layer's dgrad / wgrad GEMMs consume).  Upstream runs
 * triton_rms_norm_backward (linghe/utils/norm.py:144) and triton_blockwise_quant
 * (linghe/quant/block.py:129) as separate passes over dy. */
int lh_rmsnorm_bwd_blockquant(const void* dy, const void* x, const void* gamma, const float* rms, int dtype,
                              int64_t M, int64_t n, float eps, void* dx, float* dgamma, void* dy_q,
                              float* dy_s, void* dy_qt, float* dy_st, int round_scale, void* scratch,
                              int64_t scratch_bytes, void* stream);

/* ---- SwiGLU (dense) ------------------------------------------------------------ */

/* y = x1*sigmoid(x1)*x2 [* w_row] in the input dtype; x [M,2n], x1 = x[:, :n].
 * Replaces triton_weighted_silu_forward, linghe/utils/silu.py:98.
 * w: optional per-row weight (NULL = none), w_dtype LH_F32 or LH_BF16. */
int lh_weighted_silu_fwd(const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n, void* y,
                         void* stream);

/* Backward of the above: dx [M,2n] input dtype, dw [M] in w_dtype (when w != NULL).
 * Replaces triton_weighted_silu_backward, linghe/utils/silu.py:177. */
int lh_weighted_silu_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype, int64_t M,
                         int64_t n, void* dx, void* dw, void* stream);

/* SwiGLU + blockwise quantisation.
 * Replaces triton_silu_and_block_quant_forward, linghe/utils/silu.py:279.
 * n % 128 == 0, except mode 1 (qT, sT only), which takes n % 64 == 0 as upstream does
 * (linghe/utils/silu.py:313-317). */
int lh_silu_blockquant_fwd(const void* x, int dtype, int64_t M, int64_t n, void* q, float* s, void* qt,
                           float* st, int round_scale, int output_mode, void* stream);

/* SwiGLU backward + blockwise quantisation of dx = [dx1 | dx2]  ([M,2n]).
 * Replaces triton_silu_and_block_quant_backward, linghe/utils/silu.py:424.
 * dx_hp: optional [M,2n] copy of dx in the input dtype (NULL = none); upstream gets it
 * from a separate triton_weighted_silu_backward pass (linghe/utils/silu.py:177). */
int lh_silu_blockquant_bwd(const void* g, const void* x, int dtype, int64_t M, int64_t n, void* dx_q,
                           float* dx_s, void* dx_qt, float* dx_st, void* dx_hp, int round_scale,
                           void* stream);

/* ---- SwiGLU (per-expert batched, routed experts) ------------------------------- */

/* Replaces triton_batch_weighted_silu_and_block_quant_forward, linghe/utils/silu.py:797.
 * x [R,2n]; w [R] per-row weight (w_dtype LH_F32 / LH_BF16); counts [E] device. */
int lh_batch_silu_blockquant_fwd(const void* x, const void* w, int dtype, int w_dtype, const void* counts,
                                 int counts_type, int E, int64_t R, int64_t n, void* q, float* s, void* qt,
                                 float* st, int round_scale, int output_mode, void* stream);

/* Replaces triton_batch_weighted_silu_and_block_quant_backward, linghe/utils/silu.py:1293.
 * dw [R] in w_dtype.  scratch: lh_scratch_bytes("batch_silu_bwd", R, n) bytes. */
int lh_batch_silu_blockquant_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype,
                                 const void* counts, int counts_type, int E, int64_t R, int64_t n,
                                 void* dx_q, float* dx_s, void* dw, void* dx_qt, float* dx_st,
                                 int round_scale, void* scratch, int64_t scratch_bytes, void* stream);

/* ---- routing helpers around the permute + quantise step --------------------------- */

/* Destination row of every routed (token, expert) pair with each expert padded to a multiple of
 * `multiple_of` rows, and the inverse list of source tokens.
 * Replaces triton_make_row_id_map_and_index, linghe/utils/gather.py:161.
 * routing_map [tokens, experts]: 1-byte (bool) elements, or int32 when map_is_i32 != 0.
 * row_id_map [tokens, experts] int32 (-1 = not routed); row_index [sum of padded counts] int32: written
 * for real rows only (the caller zero-fills it, as the reference does).
 * scratch: lh_scratch_bytes("row_id_map", tokens, experts) bytes. */
int lh_make_row_id_map_and_index(const void* routing_map, int map_is_i32, int64_t tokens, int64_t experts,
                                 int multiple_of, int32_t* row_id_map, int32_t* row_index, void* scratch,
                                 int64_t scratch_bytes, void* stream);

/* out[t] = sum over experts (in expert order, float32) of grad[row_id_map[t,e]]; prob_out[t,e] =
 * probs[row_id_map[t,e]] or 0.  Replaces triton_unpermute_with_mask_map, linghe/utils/scatter.py:193.
 * grad [rows, n] in `dtype`; probs / prob_out optional (both or neither), probs_dtype LH_F32 / LH_BF16. */
int lh_unpermute_with_mask_map(const void* grad, int dtype, const int32_t* row_id_map, const void* probs,
                               int probs_dtype, int64_t tokens, int64_t experts, int64_t n, void* out,
                               void* prob_out, void* stream);

/* ---- the smooth-quant recipe: one scale per row after a per-column smoothing divisor ---- */

/* RMSNorm + smooth quantisation:  y = RMSNorm(x) * gamma;  ys = y / max(smooth_scale, 1e-30);
 * scale[r] = max(max_c |ys[r,c]| / 448, 1e-30) (rounded up to a power of two when round_scale);
 * q = e4m3(ys / scale[r]).
 * Replaces triton_rms_norm_and_smooth_quant_forward, linghe/utils/norm.py:557.
 * x [M,n] and gamma [n] of `dtype`, smooth_scale float32 [n], n <= 8192, n % 8 == 0.
 * Outputs: q e4m3 [M,n], scale float32 [M]; rms (optional) float32 [M] 1/rms per row;
 * maxs (optional, "calibrate") float32 [n] = max over rows of |y|, which needs
 * lh_scratch_bytes("smooth_quant", M, n) bytes of scratch (none otherwise). */
int lh_rmsnorm_smoothquant_fwd(const void* x, const void* gamma, const float* smooth_scale, int dtype, int64_t M,
                               int64_t n, float eps, void* q, float* scale, float* rms, float* maxs, void* scratch,
                               int64_t scratch_bytes, int round_scale, void* stream);

/* SwiGLU + smooth quantisation: y = silu(x[:, :n]) * x[:, n:], then as above.
 * Replaces triton_silu_and_smooth_quant_forward, linghe/utils/silu.py:1498.  x [M,2n]. */
int lh_silu_smoothquant_fwd(const void* x, const float* smooth_scale, int dtype, int64_t M, int64_t n, void* q,
                            float* scale, float* maxs, void* scratch, int64_t scratch_bytes, int round_scale,
                            void* stream);

/* SwiGLU backward + smooth quantisation of dx = [dx1 | dx2] on both axes.
 * Row-wise copy: dx * smooth_scale[c] (reverse != 0) or dx / max(smooth_scale[c], 1e-30), one
 * scale per row.  Transposed copy: dx[r,c] * transpose_smooth_scale[r] (or divided), one scale
 * per column of dx over all M rows.
 * Replaces triton_silu_and_smooth_quant_backward, linghe/utils/silu.py:1705.
 * g [M,n], x [M,2n] of `dtype`; smooth_scale float32 [2n], transpose_smooth_scale float32 [M];
 * outputs dx_q e4m3 [M,2n], dx_scale [M], dxt_q e4m3 [2n,M], dxt_scale [2n]; n <= 4096, n % 8 == 0;
 * scratch: lh_scratch_bytes("smooth_quant_bwd", M, n) bytes. */
int lh_silu_smoothquant_bwd(const void* g, const void* x, const float* smooth_scale, const float* transpose_smooth_scale,
                            int dtype, int64_t M, int64_t n, void* dx_q, float* dx_scale, void* dxt_q, float* dxt_scale,
                            void* scratch, int64_t scratch_bytes, int round_scale, int reverse, void* stream);

/* Per-expert weighted SwiGLU + smooth quantisation: rows grouped by expert (counts[e] rows each),
 * y = silu(x1) * x2; ys = (y * w[row]) / max(smooth_scale[e], 1e-30) (reverse != 0: * smooth_scale[e]);
 * one scale per row.  maxs (optional, "calibrate") float32 [E, n] = per-expert column maxima of
 * |y| before the weight.
 * Replaces triton_batch_weighted_silu_and_smooth_quant_forward, linghe/utils/silu.py:1821.
 * x [R,2n], w [R] (w_dtype), smooth_scale float32 [E,n], counts as in the block-format entries;
 * n <= 8192, n % 8 == 0, E <= 4096. */
int lh_batch_silu_smoothquant_fwd(const void* x, const void* w, int dtype, int w_dtype, const float* smooth_scale,
                                  const void* counts, int counts_type, int E, int64_t R, int64_t n, void* q, float* scale,
                                  float* maxs, int round_scale, int reverse, void* stream);

/* Backward of the above with smooth quantisation of dx = [dx1 | dx2] on both axes, per expert:
 * dw [R] (w_dtype); row-wise copy smoothed by smooth_scale[e] ([E,2n]), one scale per row;
 * transposed copy smoothed by transpose_smooth_scale[row] ([R]), one scale per (expert, column):
 * dxt_scale [E,2n]; expert e's transposed codes are a [2n, pad32(counts[e])] block (zero codes in
 * the padding) at byte offset 2n * sum_{e' < e} pad32(counts[e']) of dxt_q; padded_rows =
 * sum_e pad32(counts[e]).  Experts without rows get the floor scale (all zero when R == 0).
 * Replaces triton_batch_weighted_silu_and_smooth_quant_backward, linghe/utils/silu.py:2126.
 * n <= 4096, n % 8 == 0, E <= 2048. */
int lh_batch_silu_smoothquant_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype,
                                  const float* smooth_scale, const float* transpose_smooth_scale, const void* counts,
                                  int counts_type, int E, int64_t R, int64_t n, int64_t padded_rows, void* dx_q,
                                  float* dx_scale, void* dw, void* dxt_q, float* dxt_scale, int round_scale, int reverse,
                                  void* stream);

/* ---- consumer of the wire format ------------------------------------------------- */

/* Blockwise-scaled FP8 GEMM  c [M,N] = dequant(a) . dequant(b)^T.
 * Replaces triton_tt_fp8_gemm, linghe/gemm/blockwise_fp8_gemm.py:152.
 * a [M,K], b [N,K] e4m3 codes; one float32 scale per 1 x block_size run of k (block_size
 * 128 or 64; K a multiple of 128, any number of scale blocks).  Scales as the reference
 * stores them, a_s [M, K/block] and b_s [N, K/block], or -- *_transposed != 0 -- as the
 * quantisers of this library write them, [K/block, M] and [K/block, N], so that
 * (q, s) of lh_blockwise_quant / lh_rmsnorm_blockquant_fwd feed it unchanged.
 * out_dtype: LH_BF16 / LH_F16 / LH_F32. */
int lh_fp8_gemm(const void* a, const void* b, const float* a_s, const float* b_s, void* c, int64_t M, int64_t N,
                int64_t K, int block_size, int a_s_transposed, int b_s_transposed, int out_dtype, void* stream);

/* The same product with 2-D block scales: one float32 scale per block_size x block_size
 * sub-matrix, a_s [ceil(M/block), K/block] and b_s [ceil(N/block), K/block] (what
 * lh_block_quant writes for block_size 128).
 * Replaces triton_bb_fp8_gemm, linghe/gemm/blockwise_fp8_gemm.py:59. */
int lh_fp8_gemm_bb(const void* a, const void* b, const float* a_s, const float* b_s, void* c, int64_t M, int64_t N,
                   int64_t K, int block_size, int out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LINGHE_B200_H_ */
