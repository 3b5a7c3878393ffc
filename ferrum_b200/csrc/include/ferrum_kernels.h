// C launch interface of the sm_100a kernels.  Every function enqueues work on
// `stream` and returns 0 or a cudaError_t / negative argument-error code; no
// function here allocates device memory unless its comment says so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- activation / unary op codes (shared by GEMM epilogues and elementwise kernels)
enum {
  FB_ACT_NONE = 0,
  FB_ACT_RELU = 1,
  FB_ACT_GELU = 2,  // tanh approximation, constants of ferrum-nn/src/activation.rs:254-262
  FB_ACT_SILU = 3,
  FB_ACT_TANH = 4,
  FB_ACT_SIGMOID = 5,
  FB_ACT_LEAKY_RELU = 6,
  FB_ACT_ELU = 7,
  FB_UNARY_NEG = 8,
  FB_UNARY_EXP = 9,
  FB_UNARY_LOG = 10,
  FB_UNARY_SQRT = 11,
  FB_UNARY_ABS = 12,
  FB_UNARY_SIN = 13,
  FB_UNARY_COS = 14,
  FB_UNARY_POW = 15,         // x ** alpha
  FB_UNARY_ADD_SCALAR = 16,  // x + alpha
  FB_UNARY_MUL_SCALAR = 17,  // x * alpha
  FB_UNARY_RSUB_SCALAR = 18, // alpha - x
  FB_UNARY_RDIV_SCALAR = 19, // alpha / x
  FB_UNARY_AFFINE = 20,      // x * alpha + beta   (Normalize / Scale transforms)
  FB_UNARY_CLAMP = 21,       // min(max(x, alpha), beta)
};

enum { FB_BIN_ADD = 0, FB_BIN_SUB = 1, FB_BIN_MUL = 2, FB_BIN_DIV = 3, FB_BIN_POW = 4, FB_BIN_MAX = 5, FB_BIN_MIN = 6 };
enum { FB_RED_SUM = 0, FB_RED_MEAN = 1, FB_RED_MAX = 2, FB_RED_MIN = 3, FB_RED_PROD = 4 };
enum { FB_DT_F32 = 0, FB_DT_BF16 = 3 };  // values follow ferrum-core/src/dtype.rs:31-40
enum { FB_LOSS_MSE = 0, FB_LOSS_BCE = 1, FB_LOSS_L1 = 2, FB_LOSS_SMOOTH_L1 = 3 };

// ---- GEMM -----------------------------------------------------------------
// tcgen05/TMEM bf16 GEMM: out[M,N] = act(A*B^T + bias) (+= out when beta).
// lda/ldb are the row pitches (elements) of the stored matrices: a K-major
// operand is stored [rows=M|N][K], an MN-major operand is stored [rows=K][M|N].
int fb_gemm_bf16_supported(const void* a, const void* b, long long lda, long long ldb);
// out2 (optional, bf16 outputs without accumulate): receives act'(A*B^T + bias) in the layout of out, for
// blocks whose backward would otherwise re-evaluate the activation.
int fb_gemm_bf16(const void* a, const void* b, void* out, void* out2, const float* bias, int M, int N, int K,
                 long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major, int out_bf16, int act,
                 int beta, int max_ctas, int32_t* status, cudaStream_t stream);
// fp32 operands on the tensor cores as TF32 (tcgen05.mma kind::tf32), fp32 result; lda / ldb multiples of 4.
int fb_gemm_tf32(const float* a, const float* b, float* out, const float* bias, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, int a_mn_major, int b_mn_major, int act, int beta, int max_ctas,
                 int32_t* status, cudaStream_t stream);
int fb_gemm_tf32_2cta(const float* a, const float* b, float* out, const float* bias, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, int a_mn_major, int b_mn_major, int act, int beta, int max_ctas,
                 int32_t* status, cudaStream_t stream);
// CTA-pair variant (tcgen05 cta_group::2; 256 x 256 tiles on two SMs, 256 x 128 for small outputs); same
// arguments.  Returns -3 where clusters of two CTAs cannot be scheduled.  fb_gemm_bf16_2cta_pairs() = resident pairs.
int fb_gemm_bf16_2cta(const void* a, const void* b, void* out, void* out2, const float* bias, int M, int N, int K,
                      long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major, int out_bf16,
                      int act, int beta, int max_ctas, int32_t* status, cudaStream_t stream);
int fb_gemm_bf16_2cta_pairs(void);
// Timing record of the CTA-pair kernel: 4 x 64-bit words per pair (ns): MMA thread waiting for a drained accumulator,
// waiting for operands, one epilogue warp busy, whole kernel.  NULL switches it off.
void fb_gemm_bf16_2cta_set_profile(unsigned long long* buffer);
// Tiles are walked in groups of `group_m` 256-row blocks x all column blocks (default 8); returns the previous
// value, values < 1 only query.
int fb_gemm_bf16_2cta_set_group_m(int group_m);
// Batched form over batch_outer x batch_inner slices: out[s] = alpha * A[s] * B[s]^T (+= out[s] when beta).
// Each operand carries its own (outer, inner) slice strides in elements, so head-interleaved [B, S, H, D]
// activations are multiplied in place.  Slice strides of A and B must be multiples of 8 elements.
int fb_gemm_bf16_batched(const void* a, const void* b, void* out, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int batch_outer, int batch_inner, long long sa_outer, long long sa_inner,
                         long long sb_outer, long long sb_inner, long long sc_outer, long long sc_inner,
                         int a_mn_major, int b_mn_major, int out_bf16, int beta, float alpha, int32_t* status,
                         cudaStream_t stream);
// fp32 SIMT GEMM with arbitrary element strides (parity runs, odd shapes):
// out[m,n] = act(sum_k A[m*sam + k*sak] * B[k*sbk + n*sbn] + bias[n]) (+= out when beta).
int fb_gemm_f32_simt(const float* a, const float* b, float* out, const float* bias, int M, int N, int K,
                     long long sam, long long sak, long long sbk, long long sbn, long long ldc, int act, int beta,
                     int batch, long long batch_stride_a, long long batch_stride_b, long long batch_stride_c,
                     cudaStream_t stream);

// ---- elementwise ------------------------------------------------------------
int fb_unary_fwd(const void* x, void* y, long long n, int op, float alpha, float beta, int dtype,
                 cudaStream_t stream);
// dx = dy * f'(.) ; `saved` is x or y depending on the op (see elementwise.cu).
// y = x * (*scalar) with the factor read on the device (fp32 or bf16 data).
int fb_scale_by_device_scalar(const void* x, const float* scalar, void* y, long long n, int dtype,
                              cudaStream_t stream);
int fb_unary_bwd(const void* dy, const void* saved, void* dx, long long n, int op, float alpha, float beta,
                 int dtype, cudaStream_t stream);
// Broadcasting binary op over up to 6 dims; strides in elements, 0 = broadcast.
int fb_binary_fwd(const float* a, const float* b, float* out, int op, int ndim, const long long* shape,
                  const long long* stride_a, const long long* stride_b, cudaStream_t stream);
int fb_cast(const void* src, void* dst, long long n, int src_dtype, int dst_dtype, cudaStream_t stream);
int fb_transpose_2d(const void* src, void* dst, int rows, int cols, int elem_size, cudaStream_t stream);

// ---- reductions: input viewed as [outer, R, inner] --------------------------
// `scratch` (may be NULL) lets the kernel split R over several blocks when there are
// few outputs; fb_reduce_scratch_elems() says how many floats that takes (0 = none).
long long fb_reduce_scratch_elems(long long outer, long long R, long long inner);
int fb_reduce(const float* x, float* out, long long outer, long long R, long long inner, int op, float* scratch,
              long long scratch_elems, cudaStream_t stream);
int fb_arg_reduce(const float* x, long long* idx, float* val, long long outer, long long R, long long inner,
                  int is_max, cudaStream_t stream);
// Column sums of a [rows, cols] matrix (fp32 or bf16 in, fp32 out): bias gradients.
int fb_colsum(const void* x, float* out, long long rows, long long cols, int dtype, int accumulate,
              cudaStream_t stream);

// ---- normalisation ------------------------------------------------------------
// Where the wide-row kernels (shared-memory ring fed by bulk async copies) report a wait that gave up.
void fb_layernorm_set_status(int32_t* status);
// pre_act: FB_ACT_NONE or FB_ACT_GELU applied to x before normalising (fused block).
int fb_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                     long long rows, int cols, float eps, int pre_act, int dtype, cudaStream_t stream);
// stats = [3][cols]: d_gamma, d_beta, column sum of dx (accumulated into); partial = [nblk][3][cols] workspace.
// act_grad (optional, dtype of x; excludes pre_act): x holds act(z) and act_grad holds act'(z) as written by
// the producing GEMM's epilogue; dx is then the gradient of z.
int fb_layernorm_bwd(const void* dy, const void* x, const void* act_grad, const float* gamma, const float* mean,
                     const float* rstd, void* dx, float* partial, float* stats, long long rows, int cols,
                     int pre_act, int dtype, int nblk, int want_colsum, cudaStream_t stream);
int fb_layernorm_bwd_blocks(long long rows, int cols);
int fb_batchnorm_fwd(const float* x, const float* gamma, const float* beta, float* y, float* save_mean,
                     float* save_rstd, float* running_mean, float* running_var, long long rows, int cols,
                     float eps, float momentum, int training, cudaStream_t stream);
int fb_batchnorm_bwd(const float* dy, const float* x, const float* gamma, const float* save_mean,
                     const float* save_rstd, float* dx, float* dgamma, float* dbeta, long long rows, int cols,
                     cudaStream_t stream);

// ---- softmax / losses -----------------------------------------------------------
int fb_softmax_fwd(const void* x, void* y, long long rows, int cols, int log_mode, int dtype, cudaStream_t stream);
int fb_softmax_bwd(const void* dy, const void* y, void* dx, long long rows, int cols, int log_mode, int dtype,
                   cudaStream_t stream);
// Fused log-softmax + NLL over integer labels.  Writes per-row loss, and when
// dlogits != NULL the gradient (softmax - onehot) * grad_scale in `dlogits_dtype`.
int fb_ce_fwd_bwd(const void* logits, const long long* labels, float* row_loss, void* dlogits, long long rows,
                  int cols, float grad_scale, int dtype, int dlogits_dtype, cudaStream_t stream);
// Elementwise losses: sum of per-element loss into out[0] (pre-zeroed), scaled by `scale`.
int fb_loss_fwd(const float* pred, const float* target, float* out, long long n, int kind, float scale,
                cudaStream_t stream);
int fb_loss_bwd(const float* pred, const float* target, const float* gout, float* dpred, long long n, int kind,
                float scale, cudaStream_t stream);

// ---- secondary layers: recurrent gates, convolution lowering, pooling ---------
// LSTM: pre-activations xi + hh laid out [B, 4H] as (input, forget, cell, output); `gates` receives the
// activated gates for the backward pass.  dh / dc may be NULL (no gradient from that output).
int fb_lstm_gates_fwd(const float* xi, const float* hh, const float* c_prev, float* h_out, float* c_out,
                      float* gates, long long B, int H, cudaStream_t stream);
int fb_lstm_gates_bwd(const float* dh, const float* dc, const float* gates, const float* c_prev, const float* c_out,
                      float* dpre, float* dc_prev, long long B, int H, cudaStream_t stream);
// GRU: xi, hh are [B, 3H] as (reset, update, new); `saved` is [B, 4H] (r, z, n, hn).
int fb_gru_gates_fwd(const float* xi, const float* hh, const float* h_prev, float* h_out, float* saved, long long B,
                     int H, cudaStream_t stream);
int fb_gru_gates_bwd(const float* dh, const float* saved, const float* h_prev, float* dxi, float* dhh,
                     float* dh_prev, long long B, int H, cudaStream_t stream);
// Window matrix of a convolution: cols[B*Ho*Wo, C*kh*kw] (row pitch ldk elements, fp32 or bf16) and its gradient.
int fb_im2col(const float* x, void* cols, int B, int C, int H, int W, int kh, int kw, int Ho, int Wo, int sh, int sw,
              int ph, int pw, int dh, int dw, long long ldk, int out_dtype, cudaStream_t stream);
int fb_col2im(const float* dcols, float* dx, int B, int C, int H, int W, int kh, int kw, int Ho, int Wo, int sh,
              int sw, int ph, int pw, int dh, int dw, long long ldk, cudaStream_t stream);
// 2-D pooling without padding; op 0 = max (arg receives the winner's offset inside its plane), 1 = average.
int fb_pool2d_fwd(const float* x, float* y, int* arg, int B, int C, int H, int W, int kh, int kw, int Ho, int Wo,
                  int sh, int sw, int op, cudaStream_t stream);
int fb_pool2d_bwd(const float* dy, const int* arg, float* dx, int B, int C, int H, int W, int kh, int kw, int Ho,
                  int Wo, int sh, int sw, int op, cudaStream_t stream);

// ---- dropout / embedding / collate ---------------------------------------------
int fb_dropout_fwd(const void* x, void* y, uint8_t* mask, long long n, float p, unsigned long long seed,
                   unsigned long long offset, int dtype, cudaStream_t stream);
// Graph-capturable dropout: Philox offset = offset + *dev_counter; the counter advances on the stream after the launch.
int fb_dropout_fwd_dyn(const void* x, void* y, uint8_t* mask, long long n, float p, unsigned long long seed,
                       unsigned long long offset, unsigned long long* dev_counter, int dtype, cudaStream_t stream);
int fb_dropout_bwd(const void* dy, const uint8_t* mask, void* dx, long long n, float p, int dtype,
                   cudaStream_t stream);
int fb_embedding_fwd(const float* weight, const long long* idx, void* out, long long n_idx, int dim,
                     long long vocab, long long padding_idx, int out_dtype, int32_t* status, cudaStream_t stream);
// Mean over `seq` consecutive indices: out[b] = mean_s W[idx[b, s]].
int fb_embedding_meanpool_fwd(const float* weight, const long long* idx, void* out, long long batch, int seq,
                              int dim, long long vocab, int out_dtype, cudaStream_t stream);
// dW[idx[i]] += scale * dout[i / group] ; `sorted_idx/perm` come from a radix sort of idx.
int fb_embedding_bwd_sorted(const void* dout, const long long* sorted_idx, const long long* perm, float* dweight,
                            long long n_idx, int dim, int group, float scale, long long padding_idx,
                            long long vocab, int dtype, cudaStream_t stream);
// Blockwise attention forward (tcgen05, head dimension 64, bf16): out[B, Sq, H, 64] = softmax(scale q k^T) v for
// [B, H, S, 64] views given by element strides; lse (optional) [B, H, Sq].  -2: operand not describable by TMA.
int fb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int Sq, int Skv,
                     int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb, long long k_sh,
                     long long k_ss, long long v_sb, long long v_sh, long long v_ss, float scale, int causal,
                     int32_t* status, cudaStream_t stream);
// Gradients of the blockwise attention (attention_bwd.cu), D = 64 or 128: out / d_out [B, Sq, H, D] contiguous bf16, lse as
// written by fb_attention_fwd, delta = [B, H, Sq] fp32 scratch filled by the call; dq [B, Sq, H, D], dk / dv [B, Skv, H, D].
int fb_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                     const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int H, int Sq, int Skv,
                     int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb, long long k_sh, long long k_ss,
                     long long v_sb, long long v_sh, long long v_ss, float scale, int causal, int32_t* status,
                     cudaStream_t stream);
int fb_attention_bwd_map_error(void);
// Stride-1 convolution as an implicit GEMM (gemm/tcgen05_gemm.cu) over NHWC bf16 operands with channel counts padded
// to multiples of 8, its weight gradient, and the layout changes from / to NCHW fp32 (kernels/conv_layout.cu).
int fb_conv_igemm(const void* x, const void* w, void* y, const float* bias, int B, int H, int W, int Cp, int O, int kh,
                  int kw, int ph, int pw, int dh, int dw, long long ldy, int out_bf16, int32_t* status,
                  cudaStream_t stream);
int fb_conv_wgrad_splits(int B, int Ho, int Wo, int O, int Cp, int taps);
int fb_conv_wgrad(const void* dy, const void* x, float* out, int B, int H, int W, int Cp, int O, int Op, int kh, int kw,
                  int ph, int pw, int dh, int dw, int32_t* status, cudaStream_t stream);
int fb_nchw_to_nhwc_bf16(const float* x, void* y, int B, int C, long long P, int Cp, cudaStream_t stream);
int fb_nhwc_to_nchw_f32(const float* x, float* y, int B, int C, long long P, long long ld, cudaStream_t stream);
// Space-to-depth layouts that turn a strided convolution into the stride-1 case of fb_conv_igemm (conv_layout.cu).
int fb_nchw_to_s2d_nhwc_bf16(const float* x, void* z, int B, int C, int H, int W, int sh, int sw, int ph, int pw,
                             int Hz, int Wz, long long ld, cudaStream_t stream);
int fb_s2d_nhwc_to_nchw_f32(const float* z, float* x, int B, int C, int H, int W, int sh, int sw, int ph, int pw,
                            int Hz, int Wz, long long ld, cudaStream_t stream);
int fb_gather_rows(const void* src, const long long* idx, void* dst, long long n_idx, long long row_bytes,
                   long long n_rows, int32_t* status, cudaStream_t stream);

// ---- optimizers (multi-tensor; chunk tables built on the host) -------------------
typedef struct {
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale;
} fb_adam_hparams;
typedef struct {
  float lr, momentum, weight_decay, grad_scale;
  int nesterov, first_step;
} fb_sgd_hparams;
int fb_adam_flat(float* p, const float* g, float* m, float* v, void* shadow, long long n,
                 fb_adam_hparams h, cudaStream_t stream);
int fb_sgd_flat(float* p, const float* g, float* buf, void* shadow, long long n, fb_sgd_hparams h,
                cudaStream_t stream);
// Pointer-table variants: tensors[i] described by ptrs (device arrays of length ntensors).
int fb_adam_multi(float* const* p, const float* const* g, float* const* m, float* const* v,
                  void* const* shadow, const long long* sizes, int ntensors, fb_adam_hparams h,
                  cudaStream_t stream);
int fb_sgd_multi(float* const* p, const float* const* g, float* const* buf, void* const* shadow,
                 const long long* sizes, int ntensors, fb_sgd_hparams h, cudaStream_t stream);
// Graph-capturable forms: the step-dependent factors are device scalars dyn = {lr, bias_corr1, bias_corr2,
// beta1^t, beta2^t, t} (initialise to {lr, 0, 0, 1, 1, 0}); fb_optim_advance moves them one step on the stream
// before the update launches, so a captured step replays correctly.  SGD only reads dyn[0] (lr).
int fb_optim_advance(float* dyn, float beta1, float beta2, cudaStream_t stream);
int fb_adam_multi_dyn(float* const* p, const float* const* g, float* const* m, float* const* v,
                      void* const* shadow, const long long* sizes, int ntensors, fb_adam_hparams h,
                      const float* dyn, cudaStream_t stream);
int fb_sgd_multi_dyn(float* const* p, const float* const* g, float* const* buf, void* const* shadow,
                     const long long* sizes, int ntensors, fb_sgd_hparams h, const float* dyn, cudaStream_t stream);

// ---- AMP helpers -----------------------------------------------------------------
int fb_unscale_check(float* const* g, const long long* sizes, int ntensors, float inv_scale, float* found_inf,
                     cudaStream_t stream);
int fb_sumsq_multi(const float* const* g, const long long* sizes, int ntensors, float* out, cudaStream_t stream);
int fb_scale_multi(float* const* g, const long long* sizes, int ntensors, const float* total_sumsq,
                   float max_norm, float clip_value, int mode, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
