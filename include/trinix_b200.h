/*
 * trinix_b200 — C ABI of the sm_100a (B200) backend for Trinix's layer hot path: the forward of
 * the norms, int8 ops, RoPE, GLUs and attention, and the backward of the norms, GLUs and RoPE.
 *
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and
 * strides (in ELEMENTS unless a name ends in `_bytes`), enqueues work on the
 * given CUDA stream and returns a status code (0 = ok, < 0 = error). Nothing
 * here allocates device memory, synchronises the stream or throws. Arguments
 * are validated before any launch; an error code means nothing was launched.
 * The caller owns every buffer and selects the device (cudaSetDevice) first.
 *
 * Each declaration names the interface of the reference (Trinix 0.1.4, paths
 * relative to its repository root) whose device work it replaces.
 */
#ifndef TRINIX_B200_H_
#define TRINIX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRX_ABI_VERSION 1

typedef enum trx_status {
  TRX_OK = 0,
  TRX_ERR_NULL_POINTER = -1,  /* a required pointer is NULL */
  TRX_ERR_DTYPE = -2,         /* dtype code not supported by this entry point */
  TRX_ERR_SHAPE = -3,         /* negative / zero / inconsistent sizes */
  TRX_ERR_ALIGNMENT = -4,     /* pointer or stride not aligned as required */
  TRX_ERR_STRIDE = -5,        /* stride smaller than the extent it spans */
  TRX_ERR_UNSUPPORTED = -6,   /* legal request this build cannot serve (e.g. head_dim) */
  TRX_ERR_CUDA = -7,          /* the CUDA runtime/driver reported an error at launch */
  TRX_ERR_DEVICE_STATUS = -8, /* a kernel recorded a bounded-wait timeout in its status word */
  TRX_ERR_WORKSPACE = -9      /* workspace missing or too small */
} trx_status;

typedef enum trx_dtype { TRX_F32 = 0, TRX_F16 = 1, TRX_BF16 = 2 } trx_dtype;

typedef enum trx_glu_act {
  TRX_GLU_SWIGLU = 0,     /* up * silu(gate) */
  TRX_GLU_GEGLU_TANH = 1, /* up * gelu_tanh(gate) */
  TRX_GLU_REGLU = 2       /* up * max(gate, 0) */
} trx_glu_act;

/* Activation fused behind RMSNorm (trx_rmsnorm_act_fwd). */
typedef enum trx_row_act {
  TRX_ACT_MISH = 0,         /* n * tanh(softplus(n)) */
  TRX_ACT_QUICKGELU = 1,    /* n * sigmoid(1.702 n) */
  TRX_ACT_SQUARED_RELU = 2  /* max(n, 0)^2 */
} trx_row_act;

/* ABI version of the loaded library (TRX_ABI_VERSION at build time). */
int trx_version(void);

/* Static, human-readable text for a status code. */
const char* trx_status_string(int code);

/*
 * RMSNorm forward over R rows of C columns:
 *   rstd = 1/sqrt(mean(x^2) + eps);  y = round_x(w * round_x(x * rstd))
 * (the two roundings to the activation dtype follow the reference's PyTorch
 * backend, trinix/layers/norm/rmsnorm.py:70-75). `rstd_or_null` receives the
 * fp32 per-row rstd when non-NULL.
 * Replaces the launch made by TritonRMSNormFunction.forward,
 * trinix/kernels/rmsnorm_kernel.py:238-269 (kernel :9-61), reached through
 * TritonRMSNormKernel.apply, trinix/kernels/rmsnorm_kernel.py:387-389.
 */
int trx_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd_or_null, int64_t R,
                    int64_t C, int64_t x_row_stride, int64_t y_row_stride, float eps, int x_dtype,
                    int w_dtype, void* stream);

/*
 * LayerNorm forward: y = (x - mean) * rstd * w + b with biased variance.
 * `w_or_null` / `b_or_null` may be NULL (elementwise_affine=False,
 * trinix/layers/norm/layernorm.py:54-55); both share `wb_dtype`.
 * Replaces TritonLayerNormFunction.forward, trinix/kernels/layernorm_kernel.py:224-353
 * (kernel :11-67), reached through TritonLayerNormKernel.apply, :418-422.
 */
int trx_layernorm_fwd(const void* x, const void* w_or_null, const void* b_or_null, void* y,
                      float* mean_or_null, float* rstd_or_null, int64_t R, int64_t C,
                      int64_t x_row_stride, int64_t y_row_stride, float eps, int x_dtype,
                      int wb_dtype, void* stream);

/*
 * Per-row symmetric int8 quantisation:
 *   scale[r] = max|x[r,:]| / 127 (fp32, IEEE division)
 *   code     = clamp(round_half_even(x / scale), -127, 127); zero rows -> scale 0, codes 0.
 * No counterpart in the reference (it has no int8 code); the contract is the
 * "per-row symmetric int8 quantize/dequantize" configuration of this project's baseline.
 */
int trx_quant_rowwise_i8(const void* x, int8_t* codes, float* scales, int64_t R, int64_t C,
                         int64_t x_row_stride, int64_t codes_row_stride, int x_dtype,
                         void* stream);

/*
 * Inverse of trx_quant_rowwise_i8: y = round_y(float(code) * scale[r]).
 * No counterpart in the reference.
 */
int trx_dequant_rowwise_i8(const int8_t* codes, const float* scales, void* y, int64_t R, int64_t C,
                           int64_t codes_row_stride, int64_t y_row_stride, int y_dtype,
                           void* stream);

/*
 * Fused RMSNorm -> int8: quantises exactly the rows trx_rmsnorm_fwd would
 * write (after rounding to the activation dtype) without writing them.
 * No counterpart in the reference; its structure (norm, then an epilogue on
 * the row held on chip) is that of fused_rmsnorm_activation_forward_kernel,
 * trinix/kernels/fused/rmsnorm_activation_kernel.py:9-77.
 */
int trx_rmsnorm_quant_i8(const void* x, const void* w, int8_t* codes, float* scales, int64_t R,
                         int64_t C, int64_t x_row_stride, int64_t codes_row_stride, float eps,
                         int x_dtype, int w_dtype, void* stream);

/*
 * act(RMSNorm(x)): n = round(w * round(x * rstd)) as trx_rmsnorm_fwd computes it (the product is
 * rounded to the activation dtype only when w has that dtype; any other w dtype leaves it in
 * fp32, PyTorch's promotion), then y = round(act(n)), act one of TRX_ACT_*. One pass over HBM
 * instead of two.
 * Follows FastFusedRMSNormActivation._pytorch_forward,
 * trinix/layers/fused/rmsnorm_activation.py:72-86; replaces
 * TritonFusedRMSNormActivationKernel.apply, trinix/kernels/fused/rmsnorm_activation_kernel.py
 * (kernel :9-77).
 */
int trx_rmsnorm_act_fwd(const void* x, const void* w, void* y, int64_t R, int64_t C,
                        int64_t x_row_stride, int64_t y_row_stride, float eps, int act,
                        int x_dtype, int w_dtype, void* stream);

/*
 * Fused residual add + RMSNorm: s = float(x) + float(residual) (kept in fp32 on chip),
 *   y = round_x(w * round_x(s * rstd(s))); `sum_out_or_null` receives round_x(s), the new
 *   residual stream, when non-NULL.
 * Follows FastFusedResidualRMSNorm._pytorch_forward, trinix/layers/fused/residual_rmsnorm.py:66-73.
 * Replaces TritonFusedResidualRMSNormFunction.forward,
 * trinix/kernels/fused/residual_rmsnorm_kernel.py:212-248 (kernel :9-73), reached through
 * TritonFusedResidualRMSNormKernel.apply(X, Residual, W, eps).
 */
int trx_residual_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y,
                             void* sum_out_or_null, float* rstd_or_null, int64_t R, int64_t C,
                             int64_t x_row_stride, int64_t res_row_stride, int64_t y_row_stride,
                             int64_t sum_row_stride, float eps, int x_dtype, int w_dtype,
                             void* stream);

/*
 * Fused residual add + LayerNorm: s = float(x) + float(residual) (fp32, on chip),
 *   y = round(round(w * round((s - mean(s)) * rstd)) + b)  — the normalised value is cast to the
 *   activation dtype before the affine part, which runs in the parameters' dtype (a parameter
 *   dtype other than the activation's promotes to fp32 and rounds once at the end);
 *   sum_out_or_null receives round(s). w and b may be NULL.
 * Follows FastFusedResidualLayerNorm._pytorch_forward,
 * trinix/layers/fused/residual_layernorm.py:66-73; replaces
 * TritonFusedResidualLayerNormKernel.apply, trinix/kernels/fused/residual_layernorm_kernel.py
 * (kernel :9-79).
 */
int trx_residual_layernorm_fwd(const void* x, const void* residual, const void* w_or_null,
                               const void* b_or_null, void* y, void* sum_out_or_null,
                               float* mean_or_null, float* rstd_or_null, int64_t R, int64_t C,
                               int64_t x_row_stride, int64_t res_row_stride, int64_t y_row_stride,
                               int64_t sum_row_stride, float eps, int x_dtype, int w_dtype,
                               void* stream);

/*
 * Fused residual add + RMSNorm -> int8: quantises exactly the rows trx_residual_rmsnorm_fwd
 * would write, without writing them; optionally writes the summed residual stream.
 * No counterpart in the reference (it has no int8 code).
 */
int trx_residual_rmsnorm_quant_i8(const void* x, const void* residual, const void* w, int8_t* codes,
                                  float* scales, void* sum_out_or_null, int64_t R, int64_t C,
                                  int64_t x_row_stride, int64_t res_row_stride,
                                  int64_t codes_row_stride, int64_t sum_row_stride, float eps,
                                  int x_dtype, int w_dtype, void* stream);

/*
 * Rotary position embedding, half-split ("rotate_half") form, q and k in one launch:
 *   o[..., :D/2] = x1*cos - x2*sin ;  o[..., D/2:] = x2*cos + x1*sin
 * with cos/sin rows indexed by the sequence position (tables are (S, >= D/2),
 * only the first D/2 columns are read). Tensors are (B, S, H, D) with D
 * contiguous; q and k may have different head counts and arbitrary b/s/h strides.
 * `table_dtype` is TRX_F32 or equal to `x_dtype`; in the latter case every
 * intermediate product is rounded to `x_dtype` like the reference's PyTorch path
 * (trinix/layers/embeddings/rope.py:111-118). `inverse != 0` negates sin.
 * Replaces TritonRoPEFunction.forward, trinix/kernels/rope_kernel.py:165-170
 * (two launches of _rope_rotation_kernel, :11-88), reached through
 * TritonRoPEKernel.apply, :209-213.
 */
int trx_rope_fwd(const void* q, const void* k, const void* cos_table, const void* sin_table,
                 void* q_out, void* k_out, int64_t B, int64_t S, int64_t Hq, int64_t Hk, int64_t D,
                 const int64_t q_strides[3], const int64_t k_strides[3],
                 const int64_t qo_strides[3], const int64_t ko_strides[3],
                 int64_t table_row_stride, int table_dtype, int x_dtype, int inverse,
                 void* stream);

/*
 * Gated linear unit forward: y[r, c] = up[r, c] * act(gate[r, c]) for R rows of H columns.
 * `up` and `gate` are separate pointers with their own row strides so that both the
 * reference's concatenated layout (x[..., :H] = up, x[..., H:] = gate) and
 * separate tensors work.
 * Replaces TritonSwiGLUFunction.forward (trinix/kernels/swigelu_kernel.py:121-152),
 * the GeGLU forward (trinix/kernels/geglu_kernel.py:9-49) and the ReGLU forward
 * (trinix/kernels/reglu_kernel.py:9-41), reached through Triton{SwiGLU,GeGLU,ReGLU}Kernel.apply.
 */
int trx_glu_fwd(const void* up, const void* gate, void* y, int64_t R, int64_t H,
                int64_t up_row_stride, int64_t gate_row_stride, int64_t y_row_stride, int act,
                int dtype, void* stream);

/*
 * Backward of the GLUs: dup = dy * act(gate), dgate = dy * up * act'(gate), fp32 math, one
 * rounding per output. Every tensor has its own row stride, so dup / dgate may be the two halves
 * of a concatenated (R, 2H) gradient.
 * Replaces TritonSwiGLUFunction.backward (trinix/kernels/swigelu_kernel.py:154-180, kernel
 * :47-91) and the GeGLU / ReGLU backward kernels (trinix/kernels/geglu_kernel.py:53-108,
 * trinix/kernels/reglu_kernel.py:45-87).
 */
int trx_glu_bwd(const void* dy, const void* up, const void* gate, void* dup, void* dgate,
                int64_t R, int64_t H, int64_t dy_row_stride, int64_t up_row_stride,
                int64_t gate_row_stride, int64_t dup_row_stride, int64_t dgate_row_stride, int act,
                int dtype, void* stream);

/*
 * Bytes of device workspace the norm backward entry points need for R rows of C columns: two
 * (P, C) fp32 blocks of per-CTA column sums (P <= 1024, bounded so a block stays <= 16 MiB) plus
 * (R, 2) fp32 row statistics. Contents on entry are irrelevant; nothing is kept between calls.
 */
size_t trx_norm_bwd_workspace_bytes(int64_t R, int64_t C);

/*
 * RMSNorm backward. With n = x * rsqrt(mean(x^2) + eps) (recomputed from x, nothing saved by the
 * forward is needed) and g = dy * w:  dx = rstd * (g - n * mean(g * n)),  dw = sum_rows dy * n
 * (fp32 sums in a fixed order: deterministic for a given shape and device; stored in w_dtype).
 * dw_or_null == NULL skips the weight gradient.
 * Replaces TritonRMSNormFunction.backward (trinix/kernels/rmsnorm_kernel.py:270-321; kernels
 * rmsnorm_backward_dx_fused :65-147 with its lock-guarded accumulation, rmsnorm_backward_dw
 * :151-194).
 */
int trx_rmsnorm_bwd(const void* dy, const void* x, const void* w, void* dx, void* dw_or_null,
                    int64_t R, int64_t C, int64_t dy_row_stride, int64_t x_row_stride,
                    int64_t dx_row_stride, float eps, int x_dtype, int w_dtype, void* workspace,
                    size_t workspace_bytes, void* stream);

/*
 * LayerNorm backward. n = (x - mean) * rstd, g = dy * w (w == NULL: g = dy):
 *   dx = rstd * (g - mean(g) - n * mean(g * n)),  dw = sum_rows dy * n,  db = sum_rows dy.
 * dw_or_null / db_or_null == NULL skip that gradient.
 * Replaces TritonLayerNormFunction.backward (trinix/kernels/layernorm_kernel.py:298-353; kernels
 * layernorm_backward_dx_fused :71-164, layernorm_backward_dwdb :168-221).
 */
int trx_layernorm_bwd(const void* dy, const void* x, const void* w_or_null, void* dx,
                      void* dw_or_null, void* db_or_null, int64_t R, int64_t C,
                      int64_t dy_row_stride, int64_t x_row_stride, int64_t dx_row_stride, float eps,
                      int x_dtype, int wb_dtype, void* workspace, size_t workspace_bytes,
                      void* stream);

/*
 * Backward of the residual forms: the normalised row is the fp32 sum x + residual, exactly as in
 * trx_residual_rmsnorm_fwd / trx_residual_layernorm_fwd; d/dx and d/dresidual are the same tensor,
 * written once to dx. Otherwise as trx_rmsnorm_bwd / trx_layernorm_bwd (same workspace).
 * Replace TritonFusedResidualRMSNormFunction.backward
 * (trinix/kernels/fused/residual_rmsnorm_kernel.py:251-303; kernels :77-205) and
 * TritonFusedResidualLayerNormFunction.backward
 * (trinix/kernels/fused/residual_layernorm_kernel.py:278-335; kernels :83-225).
 */
int trx_residual_rmsnorm_bwd(const void* dy, const void* x, const void* residual, const void* w,
                             void* dx, void* dw_or_null, int64_t R, int64_t C,
                             int64_t dy_row_stride, int64_t x_row_stride, int64_t res_row_stride,
                             int64_t dx_row_stride, float eps, int x_dtype, int w_dtype,
                             void* workspace, size_t workspace_bytes, void* stream);
int trx_residual_layernorm_bwd(const void* dy, const void* x, const void* residual,
                               const void* w_or_null, void* dx, void* dw_or_null, void* db_or_null,
                               int64_t R, int64_t C, int64_t dy_row_stride, int64_t x_row_stride,
                               int64_t res_row_stride, int64_t dx_row_stride, float eps,
                               int x_dtype, int wb_dtype, void* workspace, size_t workspace_bytes,
                               void* stream);

/*
 * Backward of act(RMSNorm(x)) (trx_rmsnorm_act_fwd): with z = w * n the upstream gradient becomes
 * dy * act'(z), then as trx_rmsnorm_bwd (same workspace). act is one of TRX_ACT_*.
 * Replaces TritonFusedRMSNormActivationFunction.backward
 * (trinix/kernels/fused/rmsnorm_activation_kernel.py:280-330; kernels :81-233).
 */
int trx_rmsnorm_act_bwd(const void* dy, const void* x, const void* w, void* dx, void* dw_or_null,
                        int64_t R, int64_t C, int64_t dy_row_stride, int64_t x_row_stride,
                        int64_t dx_row_stride, float eps, int act, int x_dtype, int w_dtype,
                        void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of zero-initialised device workspace trx_attn_fwd needs (status word + scheduler state). */
size_t trx_attn_workspace_bytes(void);

/*
 * Attention forward, softmax(scale * Q K^T + bias) V with online softmax:
 *   q (B, Sq, Hq, D), k/v (B, Sk, Hk, D), out (B, Sq, Hq, D); D contiguous, D in {64, 128};
 *   Hq % Hk == 0, query head h reads kv head h / (Hq / Hk)  (GQA / MQA natively; a kv head
 *   stride of 0 — an expanded single head — is accepted);
 *   causal: key j visible to query i iff j <= i;
 *   window_left/right >= 0: visible iff -left <= j - i <= right (pass -1/-1 for no window);
 *   slopes_or_null: fp32 [Hq], adds -slope[h] * |i - j| after scaling (ALiBi);
 *   lse_or_null: fp32 (B, Hq, Sq) natural-log sum-exp per row, optional.
 * `workspace` points at trx_attn_workspace_bytes() bytes that were zero when first used;
 * word 0 accumulates a non-zero code if a bounded on-chip wait ever gave up.
 * strides are (batch, seq, head) in elements. dtype: TRX_BF16 or TRX_F16.
 * Replaces TritonAttentionKernel.apply, trinix/kernels/attention_kernel.py:498-664
 * (kernel _fwd_kernel, :235-434), reached through triton_attn_func,
 * trinix/layers/attention/functional.py:8-140, and the flash_attn_func call at
 * trinix/layers/attention/base.py:338-344.
 */
int trx_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse_or_null,
                 const float* slopes_or_null, int64_t B, int64_t Sq, int64_t Sk, int64_t Hq,
                 int64_t Hk, int64_t D, const int64_t q_strides[3], const int64_t k_strides[3],
                 const int64_t v_strides[3], const int64_t o_strides[3], float scale, int causal,
                 int64_t window_left, int64_t window_right, int dtype, void* workspace,
                 size_t workspace_bytes, void* stream);

/*
 * trx_attn_fwd with a dense additive mask: softmax(scale * Q K^T + mask [+ ALiBi]) V.
 *   mask: (B, Hq, Sq, Sk) values added to the scaled scores (0 keeps, -inf hides); fp32 or the
 *   activation dtype (mask_dtype); mask_strides = (batch, head, query) in elements, the key
 *   stride is 1; a batch or head stride of 0 broadcasts, which is how the reference's 2-D
 *   (Sq, Sk), 3-D (B, Sq, Sk) and 4-D (B, 1, Sq, Sk) masks are passed without expanding them.
 *   causal / window / ALiBi combine with it; a row whose keys are all hidden returns 0.
 * Every KV tile a query tile can see is visited (a dense mask gives no tile to skip), and the
 * mask is read once per score: 4 bytes per score for fp32, so the call is bound by the mask's
 * HBM traffic unless the mask is broadcast over batch and heads.
 * Replaces the attn_mask path of TritonAttentionKernel.apply,
 * trinix/kernels/attention_kernel.py:479-495 (_prepare_mask) and :9-231 (_fwd_kernel_with_mask);
 * mask semantics of FastBaseAttention._apply_pytorch_attention,
 * trinix/layers/attention/base.py:381-392.
 */
int trx_attn_fwd_mask(const void* q, const void* k, const void* v, void* out, float* lse_or_null,
                      const float* slopes_or_null, const void* mask, int mask_dtype,
                      const int64_t mask_strides[3], int64_t B, int64_t Sq, int64_t Sk, int64_t Hq,
                      int64_t Hk, int64_t D, const int64_t q_strides[3],
                      const int64_t k_strides[3], const int64_t v_strides[3],
                      const int64_t o_strides[3], float scale, int causal, int64_t window_left,
                      int64_t window_right, int dtype, void* workspace, size_t workspace_bytes,
                      void* stream);

/*
 * trx_attn_fwd_mask with dropout on the attention probabilities (mask_or_null may be NULL):
 *   out = sum_j keep_ij * P_ij / (1 - p_eff) * V_j,   P = softmax(scale * Q K^T + bias)
 * i.e. the probabilities are normalised first and dropped afterwards, the order of the reference's
 * PyTorch backend (F.dropout on the softmax output, trinix/layers/attention/base.py:394-397); the
 * LSE output is that of the undropped scores. The keep decision of element (b, h, i, j) is a pure
 * function of (seed, offset, b, h, i, j): byte (j mod 16) of Philox4x32-10 with key
 * (seed & 0xffffffff, seed >> 32) and counter (j / 16, i, b * Hq + h, offset), little-endian over
 * the four result words; the element is dropped when that byte is below
 * t = clamp(round(256 * dropout_p), 1, 255), so the realised probability is p_eff = t / 256 and
 * kept elements are scaled by 256 / (256 - t). The stream can therefore be rebuilt on the host,
 * which is how the tests check it element for element. 0 <= dropout_p < 1; 0 means no dropout.
 * Replaces the dropout branch of the reference's kernel, trinix/kernels/attention_kernel.py:395-405
 * (seed drawn at :526-532), whose own random stream (Triton's tl.rand) cannot be reproduced and
 * whose normaliser, unlike its PyTorch backend's, includes the dropped probabilities.
 */
int trx_attn_fwd_dropout(const void* q, const void* k, const void* v, void* out,
                         float* lse_or_null, const float* slopes_or_null, const void* mask_or_null,
                         int mask_dtype, const int64_t mask_strides[3], int64_t B, int64_t Sq,
                         int64_t Sk, int64_t Hq, int64_t Hk, int64_t D, const int64_t q_strides[3],
                         const int64_t k_strides[3], const int64_t v_strides[3],
                         const int64_t o_strides[3], float scale, int causal, int64_t window_left,
                         int64_t window_right, int dtype, float dropout_p, uint64_t seed,
                         uint32_t offset, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Status word of an attention workspace, read without synchronising. `host_word` is host
 * memory the caller keeps alive across calls (pinned memory keeps the copy asynchronous),
 * zero before the first call. If *host_word — as copied there by an earlier call — is already
 * non-zero, a kernel gave up on a bounded wait and every later launch on that workspace has
 * skipped its work: the call returns TRX_ERR_DEVICE_STATUS and enqueues nothing; the caller
 * zeroes the device word and *host_word before using the workspace again. Otherwise a 4-byte
 * copy of the device word into *host_word is enqueued on `stream`, behind the launches already
 * there. Call it after each trx_attn_fwd / trx_attn_fwd_mask (or every few).
 * Replaces nothing in the reference: there the failure path is the silent PyTorch fallback of
 * trinix/layers/attention/base.py:435-439.
 */
int trx_attn_status(const void* workspace, unsigned int* host_word, void* stream);

/*
 * trx_attn_fwd for callers that cannot provide a workspace. No counterpart in the reference.
 *
 * Who needs it: hosts that pass pointers in but cannot create device memory when the call is
 * made — an inference-engine plugin whose memory plan is fixed when the engine is built and
 * whose execute hook must not allocate, or a process whose device memory is owned entirely by
 * a broker. This entry point performs no cudaMalloc / cudaFree and calls no allocating library
 * routine; the kernel's 256-byte scratch block lives in a static array inside the library
 * (256 bytes on every GPU that loads the library, kept until the process exits).
 *
 * Same arguments and results as trx_attn_fwd, minus the workspace, plus
 *   status_out_or_null: optional 4-byte destination (device or pinned host memory) that
 *   receives the kernel's status word in stream order; 0 means no bounded wait gave up.
 * Limit: the static block is 256 bytes, which is what the kernel needs for EVERY problem size
 * trx_attn_fwd accepts; if the library's own requirement ever exceeds the block the call
 * returns TRX_ERR_WORKSPACE and launches nothing.
 * Arguments are checked before the block is cleared, so an argument error enqueues nothing.
 * The one error that can follow the launch is TRX_ERR_CUDA from the 4-byte copy into
 * status_out_or_null; the attention output is valid all the same.
 * The first call on each device looks up the block's device address (with that device
 * current); make that first call outside of any stream capture.
 * All calls on a device share the one block, which still holds the previous call's contents:
 * the entry point zeroes it in stream order before each launch. Two calls whose work overlaps
 * on the GPU (different streams, or different host threads feeding different streams) race
 * on it; issue them on one stream or serialise them.
 */
int trx_attn_fwd_static_scratch(const void* q, const void* k, const void* v, void* out,
                                float* lse_or_null, const float* slopes_or_null, int64_t B,
                                int64_t Sq, int64_t Sk, int64_t Hq, int64_t Hk, int64_t D,
                                const int64_t q_strides[3], const int64_t k_strides[3],
                                const int64_t v_strides[3], const int64_t o_strides[3],
                                float scale, int causal, int64_t window_left, int64_t window_right,
                                int dtype, unsigned int* status_out_or_null, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* TRINIX_B200_H_ */
