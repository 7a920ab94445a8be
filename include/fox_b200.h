/*
 * fox_b200.h -- C ABI of the B200 (sm_100a) Forgetting Attention library.
 *
 * The upstream project (zhixuan-lin/forgetting-transformer) is pure Python: its
 * operator boundary is the Python function
 *   forgetting_transformer.forgetting_attention(q, k, v, log_fgate, *, head_first,
 *       seq_start, sm_scale, adaptive_threshold)
 * (src/forgetting_transformer/ops/forgetting_attention.py:403-455) and the Triton
 * launches underneath it.  Each entry point below replaces one of those launches
 * (or the ATen call next to it) and cites the lines it stands in for.
 *
 * Conventions
 *  - every pointer is a device pointer unless stated otherwise; nothing here
 *    allocates device memory, synchronises the device or prints;
 *  - q/k/v-like tensors are logical (B, H, T, D) arrays of 16-bit floats with a
 *    unit stride on D and arbitrary element strides (sb, sh, st) on the rest,
 *    described by a fox_tensor4; base pointers and byte strides must be
 *    multiples of 16 (the Python host copies a view that is not);
 *  - (B, H, T) fp32 vectors (log_fgate, log_lambda, L, delta, dlog_lambda) are
 *    contiguous;
 *  - `dtype` is FOX_DTYPE_BF16 or FOX_DTYPE_FP16;
 *  - `stream` is a cudaStream_t passed as void*; `device` is the CUDA ordinal
 *    the buffers live on (made current for the duration of the call);
 *  - the return value is FOX_OK (0) or a negative FOX_ERR_* code.
 */
#ifndef FOX_B200_H_
#define FOX_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FOX_OK 0
#define FOX_ERR_BAD_ARG (-1)      /* null pointer, negative size, M > N ...            */
#define FOX_ERR_HEAD_DIM (-2)     /* head dim not supported by the kernel              */
#define FOX_ERR_ALIGNMENT (-3)    /* base pointer / stride not 16-byte aligned         */
#define FOX_ERR_DRIVER (-4)       /* cuTensorMapEncodeTiled entry point unavailable    */
#define FOX_ERR_TENSORMAP (-5)    /* tensor-map encoding rejected the view             */
#define FOX_ERR_LAUNCH (-6)       /* cudaGetLastError() after the launch               */
#define FOX_ERR_DEVICE (-7)       /* cudaSetDevice failed / not an sm_100 device       */
#define FOX_ERR_TOO_LARGE (-8)    /* size beyond a documented maximum                  */
#define FOX_ERR_THRESHOLD (-9)    /* reserved                                          */
#define FOX_ERR_NO_MEMORY (-10)   /* the device could not hold the library's fixed scratch array */

#define FOX_DTYPE_FP16 0
#define FOX_DTYPE_BF16 1
#define FOX_DTYPE_FP32 2          /* accepted by fox_cross_entropy_* only */

typedef struct fox_tensor4 {
  void* ptr;
  int64_t sb, sh, st; /* element strides of the B, H and T axes; D has stride 1 */
} fox_tensor4;

/* Block geometry of the attention kernels.  Adaptive Computation Pruning works on
 * whole blocks, so the index arrays below are defined relative to these sizes
 * (they play the role of get_fwd_config / get_bwd_kv_config / get_bwd_q_config,
 * forgetting_attention.py:460-493, 838-890). */
#define FOX_FWD_BLOCK_M 128
#define FOX_FWD_BLOCK_N 128
#define FOX_BWD_BLOCK_M 128
#define FOX_BWD_BLOCK_N 128

/* Library / build information: returns a static string. */
const char* fox_version(void);

/* log_lambda[b,h,t] = carry_in[b,h] + sum_{seq_start[b] <= u <= t} log_fgate[b,h,u], fp32.
 * Replaces the masked clone + torch.cumsum of forgetting_attention.py:117-127 (one pass,
 * the seq_start masking is a predicate on the load).  log_fgate may have any element
 * strides (sb, sh, sn) -- e.g. the (B,H,N) view of a (B,N,H) tensor; log_lambda is a
 * contiguous (B,H,N) array.  seq_start (B,) int64 or NULL.  carry_in (B,H) or NULL is a
 * prefix carried in from the tokens to the left (context-parallel shards); total_out
 * (B,H) or NULL receives the last prefix. */
int fox_cumsum_fwd(int device, void* stream, int64_t B, int64_t H, int64_t N, const float* log_fgate,
                   int64_t sb, int64_t sh, int64_t sn, const int64_t* seq_start, const float* carry_in,
                   float* log_lambda, float* total_out);

/* The same prefix sum straight from the gate LOGITS: log_fgate = log sigmoid(float(fgate_logit)) is formed on the
 * load, i.e. the F.logsigmoid(fgate_logit.float()) of upstream's layer (modeling_forgetting_transformer.py:343-346)
 * and the masked cumsum (forgetting_attention.py:117-127) in one pass.  fgate_logit: fp16 / bf16 / fp32 (dtype) with
 * element strides (sb, sh, sn), e.g. the (B,H,N) view of the (B,N,H) output of fgate_proj.  log_fgate_out (B,H,N)
 * fp32 or NULL receives the (unmasked) log gates. */
int fox_gate_prefix_fwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t N, const void* fgate_logit,
                        int64_t sb, int64_t sh, int64_t sn, const int64_t* seq_start, float* log_fgate_out,
                        float* log_lambda);

/* Its backward: fox_revcumsum with the chain rule through log sigmoid applied on the way out,
 * dfgate_logit[b,h,t] = sigmoid(-fgate_logit[b,h,t]) * sum_{u >= t} (dlam_col[b,h,u] + dlam_row[b,h,u-(N-M)]),
 * written in the logits' dtype with the logits' strides (sb, sh, sn). */
int fox_gate_prefix_bwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                        const float* dlam_col, const float* dlam_row, const void* fgate_logit, int64_t sb,
                        int64_t sh, int64_t sn, void* dfgate_logit);

/* dlog_fgate[b,h,t] = carry_in[b,h] + sum_{u >= t} (dlam_col[b,h,u] + dlam_row[b,h,u-(N-M)]),
 * the reverse prefix sum of forgetting_attention.py:390-392 fused with the addition of the
 * key-side and query-side halves of dlog_lambda (lines 1122, 1326-1344).  dlam_row may be NULL. */
int fox_revcumsum(int device, void* stream, int64_t B, int64_t H, int64_t M, int64_t N, const float* dlam_col,
                  const float* dlam_row, const float* carry_in, float* dlog_fgate, float* total_out);

/* Block-pruning index scans, bit-identical decisions to _find_start_index_kernel and
 * _find_end_index_kernel (forgetting_attention.py:695-745, 747-795) on a
 * (block_m, block_n) grid.  threshold is a (B,H) fp32 view with element strides
 * (thr_sb, thr_sh) (0 for broadcast axes) and must be <= 0.  start_index
 * (B,H,ceil(M/block_m)) and/or end_index (B,H,ceil(N/block_n)), int64; either may be NULL. */
int fox_find_index(int device, void* stream, int64_t B, int64_t H, int64_t M, int64_t N, int64_t block_m,
                   int64_t block_n, const float* log_lambda, const float* threshold, int64_t thr_sb,
                   int64_t thr_sh, int64_t* start_index, int64_t* end_index);

/* out[b,h] = max_t ||x[b,h,t,:]||_2 in fp32: the reduction behind adaptive_threshold="auto"
 * (torch.linalg.vector_norm(...).max(...), forgetting_attention.py:95-96).  out (B,H) fp32 must
 * be zero on entry.  D in {16,32,64,128}. */
int fox_max_row_norm(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t T, int64_t D,
                     const fox_tensor4* x, float* out_zeroed);

/* Forward attention: replaces the _fwd_kernel launch (forgetting_attention.py:186-204, kernel
 * 505-693).  q (B,H,M,D); k, v (B,H,N,D); M <= N; D in {64,128}.  log_lambda from
 * fox_cumsum_fwd.  seq_start (B,) int64 or NULL.  start_index from fox_find_index with
 * FOX_FWD_BLOCK_M/N, or NULL for no pruning.  Writes o (same dtype, caller's strides) and the
 * log-normaliser L (B,H,M) fp32 (natural log; -inf for rows left of seq_start, whose output is
 * 0).  k_norm_max: (B,H) fp32 from fox_max_row_norm(k), or NULL; with it a KV tile whose logits
 * are provably (Cauchy-Schwarz + the gate prefix) no more than 2^32 (fp16: 2^14) above the row's
 * running reference skips its row-maximum pass, which changes no result beyond fp32 rounding.
 * status: int32[4], zero on entry; [0] != 0 after the kernel means a bounded wait ran out. */
int fox_attn_fwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N, int64_t D,
                 const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const float* log_lambda,
                 const int64_t* seq_start, const int64_t* start_index, float sm_scale, const fox_tensor4* o,
                 float* L, const float* k_norm_max, int32_t* status);

/* Forward attention for ONE query row per (b,h) -- a generation step against a cache of N keys, the
 * seqlen_q = 1 case of the same upstream kernel (forgetting_attention.py:148-153, 591-693; cache:
 * fgate_cache.py:77-116).  The keys are split over `splits` CTAs per (b,h) that reduce their slice to a
 * partial (max, sum, out) triple; a second kernel merges the triples.  q, o: (B,H,1,D); k, v: (B,H,N,D),
 * 16-bit, unit inner stride, element strides multiples of 8, 16-byte aligned bases; D in {64,128};
 * log_lambda (B,H,N) from fox_cumsum_fwd; seq_start (B,) or NULL; start_index (B,H,1) or NULL; L (B,H,1)
 * fp32; workspace: fox_attn_decode_workspace_floats(B,H,D,splits) floats, fully overwritten. */
int fox_attn_decode(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t N, int64_t D,
                    const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const float* log_lambda,
                    const int64_t* seq_start, const int64_t* start_index, float sm_scale, const fox_tensor4* o,
                    float* L, float* workspace, int64_t splits);
int64_t fox_attn_decode_workspace_floats(int64_t B, int64_t H, int64_t D, int64_t splits);

/* delta[b,h,m] = sum_d o[b,h,m,d] * d_o[b,h,m,d] in fp32: replaces _bwd_preprocess
 * (forgetting_attention.py:267-277, kernel 902-943). */
int fox_bwd_delta(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t D,
                  const fox_tensor4* o, const fox_tensor4* d_o, float* delta);

/* Backward attention in one pass: replaces the _bwd_kv_kernel and _bwd_q_kernel launches
 * (forgetting_attention.py:313-334, 366-386; kernels 956-1143, 1156-1344).  end_index from
 * fox_find_index with FOX_BWD_BLOCK_M/N, or NULL.  Outputs: dk, dv (input dtype, caller's
 * strides, zero left of seq_start); dlam_col (B,H,N) fp32 = -sum_i dS_ij, fully written;
 * dq_accum_zeroed and dlam_row_zeroed may both be NULL: key side only (see fox_attn_bwd_dq; dlam_col is then the
 * sum of the fp32 dS values, as fox_attn_bwd_dq's dlam_row, instead of the 16-bit-rounded ones both sums of the
 * one-pass form are built from);
 * and two caller-provided scratch arrays that must be zero on entry and are reduced into:
 * dq_accum (B,H,M,D) fp32 = sum_j dS_ij k_j (unscaled) and dlam_row (B,H,M) fp32 = sum_j dS_ij. */
int fox_attn_bwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N, int64_t D,
                 const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o,
                 const float* log_lambda, const float* L, const float* delta, const int64_t* seq_start,
                 const int64_t* end_index, float sm_scale, float* dq_accum_zeroed, float* dlam_row_zeroed,
                 float* dlam_col, const fox_tensor4* dk, const fox_tensor4* dv, int32_t* status);

/* Query side of the backward as a kernel of its own: dq (input dtype, caller's strides, fully written) and
 * dlam_row (B,H,M) fp32 = sum_j dS_ij, fully written.  Replaces the _bwd_q_kernel launch
 * (forgetting_attention.py:366-386; kernel 1156-1344); start_index from fox_find_index with
 * FOX_BWD_BLOCK_M/N, or NULL.  Used together with fox_attn_bwd called with dq_accum_zeroed = dlam_row_zeroed =
 * NULL (key side only: dk, dv, dlam_col): at D = 128 recomputing S and dP costs less than add-reducing the
 * one-pass kernel's fp32 dQ partials into L2. */
int fox_attn_bwd_dq(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N, int64_t D,
                    const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o,
                    const float* log_lambda, const float* L, const float* delta, const int64_t* seq_start,
                    const int64_t* start_index, float sm_scale, const fox_tensor4* dq, float* dlam_row,
                    int32_t* status);

/* dq = dq_accum * scale, fp32 -> input dtype with the caller's strides (the `dq *= sm_scale`
 * and store of forgetting_attention.py:1333-1343). */
int fox_dq_convert(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t D,
                   const float* dq_accum, float scale, const fox_tensor4* dq);

/* Fused per-head RMSNorm + sigmoid gate, forward: y = x * rstd * w_h * sigmoid(g) with
 * rstd = (mean_d x^2 + eps)^-1/2 per (token, head).  Replaces layer_norm_gated_fwd
 * (fuse_norm_gate.py:539-617, kernel 132-206) for is_rms_norm, activation "sigmoid", no
 * bias/residual.  x, g, y: contiguous (tokens, G*D) 16-bit; w: (G*D) fp32; rstd: (tokens*G) fp32.
 * g == NULL leaves the gate out (y = x * rstd * w_h): the per-head RMSNorm the FoX layer applies
 * to q and k (GroupNorm(num_groups=H, is_rms_norm=True), modeling_forgetting_transformer.py:264-265,
 * 314-316; layer_norm_fwd of layernorm.py:248-325, kernel 183-245). */
int fox_normgate_fwd(int device, void* stream, int dtype, int64_t tokens, int64_t G, int64_t D, const void* x,
                     const void* g, const float* w, float eps, void* y, float* rstd);

/* Backward of the above: dx, dg (16-bit) and per-CTA partial weight gradients dw_partial
 * (n_partials, G*D) fp32, fully written, to be summed over axis 0 by the caller.  Replaces
 * layer_norm_gated_bwd (fuse_norm_gate.py:620-723, kernel 309-421).  g and dg both NULL: backward
 * of the ungated per-head RMSNorm (layer_norm_bwd, layernorm.py:426-520, kernel 328-423). */
int fox_normgate_bwd(int device, void* stream, int dtype, int64_t tokens, int64_t G, int64_t D, const void* x,
                     const void* g, const float* w, const float* rstd, const void* dy, void* dx, void* dg,
                     float* dw_partial, int64_t n_partials);

/* Row-wise RMSNorm with optional residual add, forward: z = x + residual (fp32; residual may be
 * NULL), residual_out = z rounded to the input dtype (may be NULL), rstd = (mean z^2 + eps)^-1/2,
 * y = z * rstd * w.  Replaces layer_norm_fwd with IS_RMS_NORM, a weight, no bias (layernorm.py:
 * 426-470, kernel 248-325) as RMSNorm.forward reaches it (layernorm.py:1092-1101): the FoX block's
 * attn_norm(x) and mlp_norm(x, residual, prenorm=True) (modeling_forgetting_transformer.py:565, 580).
 * x, residual, y, residual_out: contiguous (rows, hidden) 16-bit; w (hidden) fp32; rstd (rows) fp32;
 * hidden in 256 * {1,2,3,4,5,6,8}, else FOX_ERR_HEAD_DIM. */
int fox_rmsnorm_fwd(int device, void* stream, int dtype, int64_t rows, int64_t hidden, const void* x,
                    const void* residual, const float* w, float eps, void* y, void* residual_out, float* rstd);

/* Backward of the above (layer_norm_bwd, layernorm.py:473-520, kernel 328-423): z = the saved
 * residual_out (or x when there was no residual); dx = (w dy - xhat mean(xhat w dy)) rstd +
 * dresidual_in (may be NULL; the gradient that reached residual_out), which is also the gradient of
 * the residual input; dw_partial (n_partials, hidden) fp32 per-CTA partials, fully written, to be
 * summed over axis 0 by the caller. */
int fox_rmsnorm_bwd(int device, void* stream, int dtype, int64_t rows, int64_t hidden, const void* z,
                    const float* w, const float* rstd, const void* dy, const void* dresidual_in, void* dx,
                    float* dw_partial, int64_t n_partials);

/* SwiGLU, forward: z = x * sigmoid(x) * y elementwise in fp32, rounded once.  Replaces swiglu_fwd
 * (glu_linear.py:64-68; SwiGLUFunction / SwiGLULinearFunction 95-146) of ForgettingTransformerMLP
 * (modeling_forgetting_transformer.py:505-516).  x, y, z: (rows, cols) 16-bit, unit inner stride, own
 * row strides in elements (multiples of 8, >= cols): the halves of a packed projection are read in place. */
int fox_swiglu_fwd(int device, void* stream, int dtype, int64_t rows, int64_t cols, const void* x,
                   int64_t x_row_stride, const void* y, int64_t y_row_stride, void* z, int64_t z_row_stride);

/* Backward of the above (swiglu_bwd / swiglu_bwd_with_output, glu_linear.py:70-86): s = sigmoid(x);
 * dx = s (1 + x (1 - s)) g y; dy = x s g; z (may be NULL) = x s y again for the weight gradient of the
 * linear layer behind it. */
int fox_swiglu_bwd(int device, void* stream, int dtype, int64_t rows, int64_t cols, const void* x,
                   int64_t x_row_stride, const void* y, int64_t y_row_stride, const void* g, int64_t g_row_stride,
                   void* dx, int64_t dx_row_stride, void* dy, int64_t dy_row_stride, void* z, int64_t z_row_stride);

/* Cross-entropy loss per row of a (n_rows, n_cols) logit matrix, forward.  Replaces cross_entropy_fwd_kernel
 * (fused_cross_entropy.py:24-87) as FusedCrossEntropyLoss launches it for the model's loss
 * (modeling_forgetting_transformer.py:877-884), without the tensor-parallel class split:
 * z = logit_scale * logits; lse = log sum exp z; losses = lse - (1 - label_smoothing) z[label]
 * - label_smoothing * mean(z) + lse_square_scale * lse^2, and 0 where label == ignore_index; z_losses is the
 * last term alone.  logits: fp32 / bf16 / fp16 (dtype), unit inner stride, row stride in elements, rows 16-byte
 * aligned; labels int64 (n_rows); losses, z_losses, lse: fp32 (n_rows), fully written. */
int fox_cross_entropy_fwd(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols, const void* logits,
                          int64_t row_stride, const int64_t* labels, float label_smoothing, float logit_scale,
                          float lse_square_scale, int64_t ignore_index, float* losses, float* z_losses, float* lse);

/* Backward of the above (cross_entropy_bwd_kernel, fused_cross_entropy.py:90-134): dlogits = dloss * logit_scale *
 * (exp(z - lse) (1 + 2 lse_square_scale lse) - (1 - label_smoothing) [c == label] - label_smoothing / n_cols),
 * zero rows where label == ignore_index.  dlogits has the logits' dtype and may be the logits buffer itself
 * (upstream's inplace_backward); dloss: fp32 with element stride dloss_stride. */
int fox_cross_entropy_bwd(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols, const void* logits,
                          int64_t row_stride, const int64_t* labels, const float* lse, const float* dloss,
                          int64_t dloss_stride, float label_smoothing, float logit_scale, float lse_square_scale,
                          int64_t ignore_index, void* dlogits, int64_t dlogits_row_stride);

/* The same loss with the classes split over ranks (tensor parallelism over the vocabulary; replaces the
 * `process_group` path of fused_cross_entropy.py:150-151, 196-226 and :229-273).  This rank holds n_cols of
 * total_classes classes, starting at class_start.  The forward writes the rank's own log-sum-exp (lse_local) and
 * the part of the loss that needs no global one: -(1 - label_smoothing) z_label [label on this rank]
 * - label_smoothing sum_c z_c / total_classes (0 where label == ignore_index).  The host all-gathers lse_local,
 * takes their log-sum-exp, sums loss_parts over the ranks and adds the global lse (and the z-loss).  The backward
 * takes the global lse. */
int fox_cross_entropy_fwd_split(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols,
                                const void* logits, int64_t row_stride, const int64_t* labels, float label_smoothing,
                                float logit_scale, int64_t ignore_index, int64_t total_classes, int64_t class_start,
                                float* loss_parts, float* lse_local);
int fox_cross_entropy_bwd_split(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols,
                                const void* logits, int64_t row_stride, const int64_t* labels, const float* lse_global,
                                const float* dloss, int64_t dloss_stride, float label_smoothing, float logit_scale,
                                float lse_square_scale, int64_t ignore_index, int64_t total_classes,
                                int64_t class_start, void* dlogits, int64_t dlogits_row_stride);

/* Data-dependent token shift, forward: out[b,t,h,:] = x[b,t,h,:] * curr[b,t,h] + x[b,t-1,h,:] *
 * prev[b,t,h] with x[b,-1] = 0, products in fp32, rounded once.  Replaces shift_fwd_kernel
 * (token_shift.py:21-80; TokenShift.forward 164-195), which ShiftLinear calls as
 * token_shift(x, alpha, 1 - alpha) (modeling_forgetting_transformer.py:82).  x, out: (B,T,H,D)
 * 16-bit, unit stride on D, D in {16,32,64,128}, element strides (x_sb, x_st, x_sh) shared by both,
 * multiples of 8, 16-byte aligned bases; prev_weight, curr_weight: (B,T,H) fp32 sharing
 * (w_sb, w_st, w_sh). */
int fox_token_shift_fwd(int device, void* stream, int dtype, int64_t B, int64_t T, int64_t H, int64_t D,
                        const void* x, int64_t x_sb, int64_t x_st, int64_t x_sh, const float* prev_weight,
                        const float* curr_weight, int64_t w_sb, int64_t w_st, int64_t w_sh, void* out);

/* Backward of the above (shift_bwd_kernel, token_shift.py:82-157; TokenShift.backward 198-235):
 * dx[b,t,h,:] = dout[b,t,h,:] * curr[b,t,h] + dout[b,t+1,h,:] * prev[b,t+1,h];
 * dcurr[b,t,h] = sum_d dout * x[b,t];  dprev[b,t,h] = sum_d dout * x[b,t-1].  dout, dx share x's
 * strides; dprev_weight, dcurr_weight are fp32 with the weights' strides, fully written. */
int fox_token_shift_bwd(int device, void* stream, int dtype, int64_t B, int64_t T, int64_t H, int64_t D,
                        const void* x, int64_t x_sb, int64_t x_st, int64_t x_sh, const float* prev_weight,
                        const float* curr_weight, int64_t w_sb, int64_t w_st, int64_t w_sh, const void* dout,
                        void* dx, float* dprev_weight, float* dcurr_weight);

/* Backward attention that allocates nothing (no counterpart upstream, where torch allocates
 * every buffer).  For hosts that cannot obtain device memory at call time -- the GPU was
 * handed to their own arena at start-up, or their thread may not make a call that serialises
 * the device as cudaMalloc/cudaFree do.  Same inputs as fox_attn_bwd; the fp32 dQ / query-side
 * gate-gradient scratch lives in a fixed 64 MiB array inside the library, so B*H*M*(D+1) must
 * be <= fox_noalloc_scratch_floats() (2^24), else FOX_ERR_TOO_LARGE.  Also finishes the job:
 * writes dq (input dtype), dk, dv, dlam_col (B,H,N) and dlog_fgate (B,H,N) fp32.  The scratch is
 * shared by all calls on a device and is cleared on `stream` at the start of each call: calls
 * that overlap on the GPU race.  The FIRST call on a device resolves the array's address, and
 * under the CUDA runtime's default lazy module loading it is also the moment the device obtains
 * the 64 MiB (from then until exit): make that call at start-up, before the host's arena takes
 * the rest of the GPU and before any stream capture, or run with CUDA_MODULE_LOADING=EAGER so
 * that the array is placed when the library first touches the device.  FOX_ERR_NO_MEMORY: the
 * device had no room left for the array. */
int fox_attn_bwd_noalloc(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                         int64_t D, const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v,
                         const fox_tensor4* d_o, const float* log_lambda, const float* L, const float* delta,
                         const int64_t* seq_start, const int64_t* end_index, float sm_scale,
                         const fox_tensor4* dq, const fox_tensor4* dk, const fox_tensor4* dv, float* dlam_col,
                         float* dlog_fgate, int32_t* status);
int64_t fox_noalloc_scratch_floats(void);

#ifdef __cplusplus
}
#endif
#endif /* FOX_B200_H_ */
