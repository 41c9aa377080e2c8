/*
 * sgb.h - C ABI of the B200 (sm_100a) backward + gradient-synchronisation
 * kernels that replace the lang::Cuda back end of apache/singa on its
 * training backward path.
 *
 * Conventions
 *  - Every entry point returns an int status: SGB_OK (0) or a negative
 *    SGB_ERR_* code.  Nothing throws, aborts or exits.
 *  - All data pointers are DEVICE pointers unless a parameter says "host".
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *    stream, which is what singa's Context::stream is).
 *  - Calls only enqueue work; none synchronises unless documented.
 *  - No entry point allocates device memory.  Kernels that need scratch take
 *    a workspace pointer + size; the matching *_workspace_bytes() query gives
 *    the requirement.  (The communicator owns its staging buffers, allocated
 *    once at creation, as the reference's does.)
 *  - Sizes are size_t element counts.  n == 0 is legal and a no-op.
 *  - Each declaration cites the reference interface (file:line inside
 *    apache/singa) that it stands in for.
 */
#ifndef SGB_H_
#define SGB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
#define SGB_OK 0
#define SGB_ERR_NULL (-1)        /* a required pointer is NULL */
#define SGB_ERR_SIZE (-2)        /* inconsistent or out-of-range size/shape */
#define SGB_ERR_CUDA (-3)        /* CUDA runtime error, see sgb_last_cuda_error */
#define SGB_ERR_WORKSPACE (-4)   /* workspace missing, too small or misaligned */
#define SGB_ERR_NCCL (-5)        /* NCCL error, see sgb_last_nccl_error */
#define SGB_ERR_UNSUPPORTED (-6) /* enum value / dtype / mode not supported */
#define SGB_ERR_STATE (-7)       /* call not valid in the handle's state */
#define SGB_ERR_CAPACITY (-8)    /* does not fit the communicator's buffers */
#define SGB_ERR_LIMIT (-9)       /* size exceeds an entry point's built-in scratch */

const char *sgb_status_string(int status);
int sgb_last_cuda_error(void); /* last cudaError_t recorded by this library */
int sgb_version(void);
/* Library-wide switches, read at launch time (set them before capturing a
 * CUDA graph; a captured launch keeps the setting it was captured with).
 * SGB_OPT_OVERLAP_LAUNCHES (default 1): the batch-norm and elementwise
 * kernels are launched with programmatic stream serialisation, so that a
 * kernel's CTAs are scheduled while the previous kernel of the same stream
 * drains; each such kernel waits for its predecessors' completion before its
 * first access to global memory, so results and stream-order semantics are
 * unchanged.  0 restores plain launches. */
enum sgb_option { SGB_OPT_OVERLAP_LAUNCHES = 1, SGB_OPT_COUNT_ = 2 };
int sgb_set_option(int option, int value);
int sgb_get_option(int option);

/* --------------------------------------------------------------- ReLU path */
/* y = x > 0 ? x : 0.  Replaces singa::cuda::relu
 * (src/core/tensor/math_kernel.h:79-80, math_kernel.cu:235-251) behind
 * ReLU<float|half, lang::Cuda> (src/core/tensor/tensor_math_cuda.h:708-720). */
int sgb_relu_f32(const float *x, float *y, size_t n, void *stream);
int sgb_relu_f16(const void *x, void *y, size_t n, void *stream);

/* dx = x > 0 ? dy : 0 (fp16: x >= 0, the reference's rule for half).
 * Replaces singa::cuda::relubackward (math_kernel.h:108-112,
 * math_kernel.cu:253-271) behind ReLUBackward<T, lang::Cuda>
 * (tensor_math_cuda.h:655-673). */
int sgb_relu_backward_f32(const float *dy, const float *x, float *dx, size_t n,
                          void *stream);
int sgb_relu_backward_f16(const void *dy, const void *x, void *dx, size_t n,
                          void *stream);

/* Fused gradient join + ReLU backward: dx = x > 0 ? (dy_a + dy_b) : 0.
 * One pass for the pair "dxs_[y_idx] += dx" (python/singa/autograd.py:204 ->
 * cuda::add) followed by ReLUBackward on the joined gradient. */
int sgb_add_relu_backward_f32(const float *dy_a, const float *dy_b,
                              const float *x, float *dx, size_t n,
                              void *stream);

/* ReLU with a one-bit-per-element record - a forward partner (it changes what
 * the backward pass consumes, so it is opt-in): y = max(x, 0) and bit i & 31
 * of 32-bit word i >> 5 of `mask` = (x[i] > 0), the rule of cuda::relubackward
 * (math_kernel.cu:253-259).  `mask` holds sgb_relu_mask_bytes(n) bytes (the
 * record rounded up to whole 16-byte groups; the backward forms may read the
 * padding, never interpret it), 4-byte aligned.  The three backward forms read the record instead of the stored
 * input (1/32 of its bytes) and give bit-identical results:
 *   relu_backward_mask      dx = bit ? dy : 0
 *   add_relu_backward_mask  dx = bit ? dy_a + dy_b : 0      (join + ReLU)
 *   bn_relu_backward_mask   batch-norm backward of dy masked by the record
 *                           (declared with the batch-norm functions). */
size_t sgb_relu_mask_bytes(size_t n);
int sgb_relu_forward_mask_f32(const float *x, float *y, void *mask, size_t n,
                              void *stream);
int sgb_relu_backward_mask_f32(const float *dy, const void *mask, float *dx,
                               size_t n, void *stream);
int sgb_add_relu_backward_mask_f32(const float *dy_a, const float *dy_b,
                                   const void *mask, float *dx, size_t n,
                                   void *stream);

/* ----------------------------------------------------- elementwise families */
/* out = a (op) b, tensor (op) tensor.  Replaces singa::cuda::add/sub/mult/
 * div/pow and gt/ge/eq/lt/le pair forms (math_kernel.h:114-166).  Comparisons
 * write 1.0f / 0.0f.  `out` may alias `a` or `b`. */
enum sgb_binary_op {
  SGB_ADD = 0, SGB_SUB = 1, SGB_MUL = 2, SGB_DIV = 3, SGB_POW = 4,
  SGB_GT = 5, SGB_GE = 6, SGB_EQ = 7, SGB_LT = 8, SGB_LE = 9
};
int sgb_binary_f32(int op, const float *a, const float *b, float *out, size_t n,
                   void *stream);
/* fp16: ADD, SUB, MUL, DIV, POW only (math_kernel.h:146-166 half overloads). */
int sgb_binary_f16(int op, const void *a, const void *b, void *out, size_t n,
                   void *stream);

/* out = in (op) x, tensor (op) scalar.  Replaces the scalar overloads
 * (math_kernel.h:84-106, 114-140).  SGB_RDIV is x / in (cuda::div with a
 * leading scalar); SGB_THRESHOLD is in < x ? 1 : 0 (cuda::threshold). */
enum sgb_scalar_op {
  SGB_S_ADD = 0, SGB_S_MUL = 1, SGB_S_RDIV = 2, SGB_S_POW = 3,
  SGB_S_GT = 4, SGB_S_GE = 5, SGB_S_EQ = 6, SGB_S_LT = 7, SGB_S_LE = 8,
  SGB_S_THRESHOLD = 9
};
int sgb_scalar_f32(int op, const float *in, float x, float *out, size_t n,
                   void *stream);
/* fp16 scalar multiply (math_kernel.h:92-93). */
int sgb_scalar_mul_f16(const void *in, float x, void *out, size_t n,
                       void *stream);

/* out = f(in).  Replaces the one-input launchers (math_kernel.h:43-82). */
enum sgb_unary_op {
  SGB_ABS = 0, SGB_SIGN, SGB_EXP, SGB_ERF, SGB_CEIL, SGB_FLOOR, SGB_ROUND,
  SGB_ROUNDE, SGB_LOG, SGB_SQRT, SGB_SQUARE, SGB_COS, SGB_COSH, SGB_ACOS,
  SGB_ACOSH, SGB_SIN, SGB_SINH, SGB_ASIN, SGB_ASINH, SGB_TAN, SGB_TANH,
  SGB_ATAN, SGB_ATANH, SGB_SIGMOID, SGB_SOFTPLUS, SGB_SOFTSIGN,
  SGB_UNARY_COUNT
};
int sgb_unary_f32(int op, const float *in, float *out, size_t n, void *stream);

/* out = min(max(in, low), high) (cuda::clamp, math_kernel.h:84-85). */
int sgb_clamp_f32(float low, float high, const float *in, float *out, size_t n,
                  void *stream);

/* Fill.  Replaces Set<float, lang::Cuda> (tensor_math_cuda.h:210-216,
 * cudnnSetTensor) and cuda::set (math_kernel.h:41); the fp16 form replaces
 * the host-vector copy of Set<half> (tensor_math_cuda.h:218-223). */
int sgb_set_f32(float v, float *out, size_t n, void *stream);
int sgb_set_f16(float v, void *out, size_t n, void *stream);

/* Casts.  Replace cuda::float2half / half2float (math_kernel.h:176-178,
 * round-to-nearest-even) and cast_float_2_int / cast_int_2_float
 * (math_kernel.h:51-54, C truncation) behind CastCopy<..., lang::Cuda>
 * (tensor_math_cuda.h:176-208). */
int sgb_cast_f32_f16(const float *in, void *out, size_t n, void *stream);
int sgb_cast_f16_f32(const void *in, float *out, size_t n, void *stream);
int sgb_cast_f32_i32(const float *in, int32_t *out, size_t n, void *stream);
int sgb_cast_i32_f32(const int32_t *in, float *out, size_t n, void *stream);
/* fp16 -> fp32 with a multiply by `scale` after widening (two roundings, as
 * half2float followed by EltwiseMult): the "cast back and scale by 1/world"
 * of the fp16 synchronisation. */
int sgb_cast_f16_f32_scaled(const void *in, float scale, float *out, size_t n,
                            void *stream);

/* y += alpha * x.  Replaces Axpy<float, lang::Cuda> (tensor_math_cuda.h:
 * 1031-1049, cublasSaxpy / cublasAxpyEx); alpha_dev is a device scalar (the
 * reference's tensor-alpha overload). */
int sgb_axpy_f32(float alpha, const float *x, float *y, size_t n, void *stream);
int sgb_axpy_dev_alpha_f32(const float *alpha_dev, const float *x, float *y,
                           size_t n, void *stream);
/* fp16 data, fp32 alpha and arithmetic, one rounding per element
 * (Axpy<half, lang::Cuda>, tensor_math_cuda.h:1051-1071, cublasAxpyEx). */
int sgb_axpy_f16(float alpha, const void *x, void *y, size_t n, void *stream);
int sgb_axpy_dev_alpha_f16(const float *alpha_dev, const void *x, void *y,
                           size_t n, void *stream);

/* BLAS-1 reductions with the result in DEVICE memory (capturable, no host
 * round trip) and a fixed summation order.  They stand in for the cuBLAS
 * calls of Dot / Asum / Nrm2 / Amax / Amin<float, lang::Cuda>
 * (tensor_math_cuda.h:1001-1029, 1075-1102).  amax / amin write the 0-based
 * index of the first element with the largest / smallest |x| (the reference
 * subtracts 1 from cublasIsamax / Isamin).  Workspace: query below. */
size_t sgb_blas1_workspace_bytes(size_t n);
int sgb_dot_f32(const float *x, const float *y, float *out, size_t n, void *ws,
                size_t ws_bytes, void *stream);
int sgb_asum_f32(const float *x, float *out, size_t n, void *ws,
                 size_t ws_bytes, void *stream);
int sgb_nrm2_f32(const float *x, float *out, size_t n, void *ws,
                 size_t ws_bytes, void *stream);
int sgb_amax_f32(const float *x, int32_t *index_out, size_t n, void *ws,
                 size_t ws_bytes, void *stream);
int sgb_amin_f32(const float *x, int32_t *index_out, size_t n, void *ws,
                 size_t ws_bytes, void *stream);
/* Row-major M (nrow x ncol): out = M * diag(v) when side_right, else
 * diag(v) * M (DGMM<float, lang::Cuda>, tensor_math_cuda.h:1112-1129). */
int sgb_dgmm_f32(int side_right, const float *M, const float *v, float *out,
                 size_t nrow, size_t ncol, void *stream);

/* Strided gather out[i] = in[offset(i)] over an nDim-dimensional shape/stride
 * (element strides; 0 = broadcast).  Replaces cuda::traverse_unary_transform
 * (math_kernel.h:95-100) behind Transform<T, lang::Cuda>
 * (tensor_math_cuda.h:238-298).  shape/stride are HOST arrays, nDim <= 8:
 * they travel as kernel arguments, so no host-to-device copy is issued. */
int sgb_strided_copy_f32(const float *in, float *out, size_t n, int nDim,
                         const int *shape_host, const int *stride_host,
                         void *stream);
int sgb_strided_copy_f16(const void *in, void *out, size_t n, int nDim,
                         const int *shape_host, const int *stride_host,
                         void *stream);
/* The inverse: out[offset(i)] = in[i], shape/stride describing `out` (no
 * broadcast dimension).  Used where the reference lets an elementwise op
 * write into a transposed view through a strided cuDNN output descriptor
 * (tensor_math_cuda.h:300-330, e.g. Exp into Transpose(x)). */
int sgb_strided_scatter_f32(const float *in, float *out, size_t n, int nDim,
                            const int *shape_host, const int *stride_host,
                            void *stream);
/* The same gather with shape/stride in DEVICE memory - the literal calling
 * convention of cuda::traverse_unary_transform (math_kernel.h:95-100), for an
 * adapter that keeps that signature. */
int sgb_strided_copy_dev_f32(const float *in, float *out, size_t n, int nDim,
                             const int *shape_dev, const int *stride_dev,
                             void *stream);
int sgb_strided_copy_dev_f16(const void *in, void *out, size_t n, int nDim,
                             const int *shape_dev, const int *stride_dev,
                             void *stream);

/* Sparsification helpers with the reference's exact semantics
 * (math_kernel.h:180-186; math_kernel.cu:628-650):
 *   sparsabs:      out = |in| >= thr ? in : 0
 *   sparsindex:    out = in == 0 ? 0 : i + 1        (1-based, int32)
 *   generateindex: out = i + 1 */
int sgb_sparsabs_f32(float thr, const float *in, float *out, size_t n,
                     void *stream);
int sgb_sparsindex_f32(const float *in, int32_t *out, size_t n, void *stream);
int sgb_generateindex_i32(int32_t *out, size_t n, void *stream);

/* ------------------------------------------------------------- reductions */
/* SumRows: v[c] = sum over rows of M[r][c], M row-major nrow x ncol - the
 * bias-gradient reduction.  Replaces SumRows (src/core/tensor/tensor.cc:
 * 1523-1538: ones vector + cudnnSetTensor + transposed cublasSgemv via
 * GEMV<float, lang::Cuda>, tensor_math_cuda.h:1129-1146).  Workspace: see
 * sgb_sum_rows_workspace_bytes (0 for most shapes); sizes depend on the SM
 * count of the current device. */
size_t sgb_sum_rows_workspace_bytes(size_t nrow, size_t ncol);
int sgb_sum_rows_f32(const float *M, float *v, size_t nrow, size_t ncol,
                     void *ws, size_t ws_bytes, void *stream);
/* SumColumns: v[r] = sum over columns of M[r][c] (tensor.cc:1508-1522). */
int sgb_sum_columns_f32(const float *M, float *v, size_t nrow, size_t ncol,
                        void *stream);
/* RowMax seeded with the first element (cuda::RowMax, math_kernel.h:173-174,
 * math_kernel.cu:488-499). */
int sgb_row_max_f32(const float *M, float *v, size_t nrow, size_t ncol,
                    void *stream);
/* Convolution bias gradient db[c] = sum_{n,h,w} dy[n][c][h][w] (NCHW,
 * HW = H*W).  Replaces GpuConvBackwardb (src/model/operation/convolution.cc:
 * 684-702, cudnnConvolutionBackwardBias). */
size_t sgb_conv_bias_backward_workspace_bytes(int N, int C, int HW);
int sgb_conv_bias_backward_f32(const float *dy, float *db, int N, int C, int HW,
                               void *ws, size_t ws_bytes, void *stream);
/* SumAll: out[0] = sum of x (device scalar).  Replaces SumAll
 * (tensor.cc:1242-1254: ones tensor + Dot<float, lang::Cuda>,
 * tensor_math_cuda.h:1084-1094). */
size_t sgb_sum_all_workspace_bytes(size_t n);
int sgb_sum_all_f32(const float *x, float *out, size_t n, void *ws,
                    size_t ws_bytes, void *stream);

/* --------------------------------------------------- softmax / cross entropy */
/* Row softmax exp(x - rowmax) / sum; y may alias x.  Replaces
 * SoftMax<float, lang::Cuda> (tensor_math_cuda.h:1274-1305,
 * CUDNN_SOFTMAX_ACCURATE / MODE_INSTANCE). */
int sgb_softmax_rows_f32(const float *x, float *y, size_t nrow, size_t ncol,
                         void *stream);
/* loss[i] = -log(max(p[i][t[i]], FLT_MIN)) (int_target) or the normalised
 * weighted sum for a batch x dim int32 target array.  Replaces
 * cuda::ComputeCrossEntropy (math_kernel.h:160-162) behind
 * ComputeCrossEntropy<float, lang::Cuda> (tensor_math_cuda.h:1375-1397). */
int sgb_cross_entropy_f32(int int_target, size_t batch, size_t dim,
                          const float *p, const int32_t *t, float *loss,
                          void *stream);
/* grad = p - target.  Same argument list as cuda::SoftmaxCrossEntropyBwd
 * (math_kernel.h:166-168; SoftmaxCrossEntropyBwd<float, lang::Cuda>,
 * tensor_math_cuda.h:1399-1425); grad may alias p (the reference edits a
 * clone of p in place) or be a separate buffer (saves the clone). */
int sgb_softmax_cross_entropy_bwd_f32(int int_target, size_t batch, size_t dim,
                                      const float *p, const int32_t *t,
                                      float *grad, void *stream);
/* grad = (p - target) * scale: the pair SoftmaxCrossEntropyBwd + "dx /= N"
 * of python/singa/autograd.py:1319-1322 in one pass (scale = 1/N as fp32). */
int sgb_softmax_cross_entropy_grad_f32(int int_target, size_t batch, size_t dim,
                                       const float *p, const int32_t *t,
                                       float scale, float *grad, void *stream);

/* The loss head of python/singa/autograd.py:1306-1322 (SoftMax, CrossEntropyFwd,
 * SoftmaxCrossEntropyBwd, "dx /= N") for integer targets in ONE launch:
 *   prob = softmax(logits) (optional, may be NULL), loss[i] = -log(max(prob[i,
 *   t[i]], FLT_MIN)), grad = (prob - onehot(t)) * scale.
 * Bit-identical to sgb_softmax_rows_f32 + sgb_cross_entropy_f32 +
 * sgb_softmax_cross_entropy_grad_f32. */
int sgb_softmax_cross_entropy_fused_f32(const float *logits, const int32_t *t,
                                        size_t batch, size_t dim, float scale,
                                        float *prob, float *loss, float *grad,
                                        void *stream);

/* fp16 forms.  Softmax computes in fp32 and rounds once on store.  The two
 * cross-entropy kernels keep the half-precision arithmetic of the overloads
 * they replace (math_kernel.cu:500-537, 588-611): probabilities floored at
 * half(1e-7), weights converted with round-down, loss and grad in __half. */
int sgb_softmax_rows_f16(const void *x, void *y, size_t nrow, size_t ncol,
                         void *stream);
int sgb_cross_entropy_f16(int int_target, size_t batch, size_t dim,
                          const void *p, const int32_t *t, void *loss,
                          void *stream);
int sgb_softmax_cross_entropy_bwd_f16(int int_target, size_t batch, size_t dim,
                                      const void *p, const int32_t *t,
                                      void *grad, void *stream);

/* --------------------------------------------------- batch-norm backward */
/* Training-mode backward from the saved batch mean and saved INVERSE standard
 * deviation (what the reference's forward stores in its `var` tensor).
 * Spatial mode: x, dy, dx are N x C x HW (NCHW); per-activation mode (2-D
 * N x D input): pass C = D, HW = 1.  dscale/dbias have C elements; dx may
 * alias dy.  Replaces GpuBatchNormBackward (src/model/operation/batchnorm.cc:
 * 368-404, cudnnBatchNormalizationBackward with alpha=1, beta=0).  Workspace
 * (16-byte aligned): sgb_bn_backward_workspace_bytes. */
size_t sgb_bn_backward_workspace_bytes(int N, int C, int HW);
int sgb_bn_backward_f32(const float *x, const float *dy, const float *scale,
                        const float *mean, const float *invstd, float *dx,
                        float *dscale, float *dbias, int N, int C, int HW,
                        void *ws, size_t ws_bytes, void *stream);
/* Gradient join + ReLU backward + batch-norm backward in one pass:
 *   joined = relu_in > 0 ? (dy_a + dy_b) : 0        (also written out: the
 *            shortcut branch of a residual block reads it)
 *   (dx, dscale, dbias) = batch-norm backward of `joined`
 * Equals sgb_add_relu_backward_f32 followed by sgb_bn_backward_f32 bit for
 * bit in `joined`, and within rounding of the sums elsewhere; it saves one
 * read of the joined gradient (the sequence "+=" join (autograd.py:204),
 * ReLUBackward, GpuBatchNormBackward at the end of every residual block). */
int sgb_bn_add_relu_backward_f32(const float *x, const float *dy_a,
                                 const float *dy_b, const float *relu_in,
                                 const float *scale, const float *mean,
                                 const float *invstd, float *joined, float *dx,
                                 float *dscale, float *dbias, int N, int C,
                                 int HW, void *ws, size_t ws_bytes,
                                 void *stream);
/* Forward partner: training-mode batch norm.  y = scale * (x - mean) * invstd
 * + bias with batch statistics; save_mean / save_invstd (= 1/sqrt(biased var
 * + eps)) are what sgb_bn_backward_f32 consumes; running_mean / running_var
 * are updated in place as r = (1 - factor) * r + factor * batch value, the
 * variance unbiased.  Replaces GpuBatchNormForwardTraining
 * (src/model/operation/batchnorm.cc:287-329, cudnnBatchNormalizationForward
 * Training; the reference passes eps = CUDNN_BN_MIN_EPSILON).  HW = 1 is the
 * per-activation mode.  Workspace as for the backward. */
int sgb_bn_forward_training_f32(const float *x, const float *scale,
                                const float *bias, float *running_mean,
                                float *running_var, float factor, float eps,
                                float *y, float *save_mean, float *save_invstd,
                                int N, int C, int HW, void *ws, size_t ws_bytes,
                                void *stream);
/* Diagnostic for the streaming form of the batch-norm backward kernels, whose
 * CTAs meet through counters in device memory with bounded waits: *flags
 * receives the sticky fault word of the current device (0 = none; bit 0 a
 * wait ran out, bit 1 a counter table was still in use by another launch - at
 * most eight such launches may be in flight per device).  A faulted launch
 * stops early and its outputs are undefined.  Synchronises the device. */
int sgb_bn_backward_faults(unsigned *flags);
/* How the streaming form would cut an (N, C, HW) problem (host arithmetic
 * only, no device work): returns 1 and fills plan6 = {pieces per plane, floats
 * per piece, pieces per item, items per channel, CTAs per SM, staged tensors
 * per item}, or 0 when the streaming form does not apply (it is used for
 * channels that do not fit a thread-block cluster).  mask: 0 none, 1 ReLU
 * input, 2 ReLU bit record. */
int sgb_bn_backward_stream_plan(int N, int C, int HW, int mask, int *plan6);
/* Batch-norm backward for callers that can neither allocate device memory nor
 * hand in a workspace.  (No counterpart in the reference: this entry point
 * exists only in this library.)  Typical callers: an operator running inside
 * a framework whose own pool already holds the device's memory, so that a
 * second allocator may fail; or a thread that must not trigger the
 * device-wide synchronisation a cudaMalloc/cudaFree can imply.  Same
 * arithmetic and results contract as sgb_bn_backward_f32 (it always takes the
 * two-pass form, so sums may differ from the other entry point in the last
 * bits).  The partial sums live in a 2 MiB array inside the library's device
 * image (held by every GPU that loads the library until exit), which limits
 * C to 4096 channels: a larger C returns SGB_ERR_LIMIT and launches
 * nothing.  No cudaMalloc/cudaFree or allocating routine is called.  The
 * first call on each device looks up the array's device address (one
 * cudaGetSymbolAddress): make that first call before any stream capture
 * begins.  All calls share the one array and it keeps the previous call's
 * contents; nothing in it needs clearing (each call overwrites every entry it
 * later reads), but two calls whose kernels can overlap on the GPU (different
 * streams, no ordering between them) race on it - keep them ordered. */
int sgb_bn_backward_noalloc_f32(const float *x, const float *dy,
                                const float *scale, const float *mean,
                                const float *invstd, float *dx, float *dscale,
                                float *dbias, int N, int C, int HW,
                                void *stream);
/* Same with the backward of the ReLU that follows the BN layer folded in:
 * dy is first masked by relu_in > 0 (relu_in = the tensor ReLU stored, i.e.
 * the BN output).  Equals ReLUBackward + GpuBatchNormBackward bit for bit. */
/* As sgb_bn_relu_backward_f32 with the ReLU decisions taken from the bit
 * record of sgb_relu_forward_mask_f32 (element order of the NCHW tensor). */
int sgb_bn_relu_backward_mask_f32(const float *x, const float *dy,
                                  const void *relu_mask, const float *scale,
                                  const float *mean, const float *invstd,
                                  float *dx, float *dscale, float *dbias, int N,
                                  int C, int HW, void *ws, size_t ws_bytes,
                                  void *stream);
int sgb_bn_relu_backward_f32(const float *x, const float *dy,
                             const float *relu_in, const float *scale,
                             const float *mean, const float *invstd, float *dx,
                             float *dscale, float *dbias, int N, int C, int HW,
                             void *ws, size_t ws_bytes, void *stream);

/* ------------------------------------------------------------------ pooling */
/* Output extent (src/model/operation/pooling.cc:46-51). */
int sgb_pool_out_size(int in, int kernel, int pad, int stride);
/* Forward partners (GpuPoolingForward, pooling.cc:180-205). */
int sgb_maxpool_forward_f32(const float *x, float *y, int N, int C, int H,
                            int W, int kh, int kw, int ph, int pw, int sh,
                            int sw, void *stream);
int sgb_avgpool_forward_f32(const float *x, float *y, int N, int C, int H,
                            int W, int kh, int kw, int ph, int pw, int sh,
                            int sw, void *stream);
/* Replaces GpuPoolingBackward (pooling.cc:207-226, cudnnPoolingBackward with
 * y, dy, x).  Max: each window's dy goes to its FIRST maximum in raster
 * order; avg: dy / (window cells inside the image).  Deterministic gather. */
int sgb_maxpool_backward_f32(const float *x, const float *y, const float *dy,
                             float *dx, int N, int C, int H, int W, int kh,
                             int kw, int ph, int pw, int sh, int sw,
                             void *stream);
int sgb_avgpool_backward_f32(const float *dy, float *dx, int N, int C, int H,
                             int W, int kh, int kw, int ph, int pw, int sh,
                             int sw, void *stream);

/* Arg-max forward partner (no reference counterpart as an interface; the
 * reference recomputes the winners from x and y inside cudnnPoolingBackward).
 * The forward also writes one byte per window: where its first maximum in
 * raster order sits, (row offset << 4) | column offset from the window's
 * unclipped corner (0xff: no cell).  The backward then reads only dy and that
 * record - results identical to sgb_maxpool_backward_f32 bit for bit.
 * kh, kw <= 15. */
int sgb_maxpool_forward_argmax_f32(const float *x, float *y,
                                   unsigned char *argmax, int N, int C, int H,
                                   int W, int kh, int kw, int ph, int pw,
                                   int sh, int sw, void *stream);
int sgb_maxpool_backward_argmax_f32(const float *dy,
                                    const unsigned char *argmax, float *dx,
                                    int N, int C, int H, int W, int kh, int kw,
                                    int ph, int pw, int sh, int sw,
                                    void *stream);

/* ------------------------------------------------- SGD update, multi-tensor */
/* One fused pass of SGD.apply (python/singa/opt.py:269-310) over p, g, m:
 *   g *= grad_scale (DistOpt.update's grad /= world, opt.py:738-746)
 *   g += weight_decay * p ; m = m * momentum ; m += (1 - dampening) * g
 *   p += -lr * (nesterov ? g + momentum * m : m)
 * each step rounded once like the BLAS-1 call it replaces (Axpy<float,
 * lang::Cuda>, tensor_math_cuda.h:1031-1049).  momentum == 0 skips m
 * (moment may be NULL).  g is read only; its reference post-state is not
 * produced.  params/grads/moments/sizes are HOST arrays of `count` entries. */
int sgb_sgd_update_f32(float *param, const float *grad, float *moment, size_t n,
                       float lr, float momentum, float dampening,
                       float weight_decay, int nesterov, float grad_scale,
                       void *stream);
int sgb_sgd_update_multi_f32(void *const *params, void *const *grads,
                             void *const *moments, const size_t *sizes,
                             size_t count, float lr, float momentum,
                             float dampening, float weight_decay, int nesterov,
                             float grad_scale, void *stream);

/* ------------------------------------------------ bucket pack / unpack */
/* Gather a HOST list of fp32 tensors into a flat device buffer starting at
 * element flat_offset, back to back (the per-tensor cudaMemcpyAsync loop of
 * Communicator::fusedSynch, src/io/communicator.cc:235-253), optionally
 * rounding to fp16 on the way (fusedSynchHalf's copy + float2half passes,
 * communicator.cc:351-370).  Unpack is the reverse (communicator.cc:281-300,
 * 393-412) with an optional multiply by `scale` after widening. */
int sgb_pack_f32(void *const *tensors, const size_t *sizes, size_t count,
                 float *flat, size_t flat_offset, void *stream);
int sgb_pack_f32_to_f16(void *const *tensors, const size_t *sizes, size_t count,
                        void *flat_f16, size_t flat_offset, void *stream);
int sgb_unpack_f32(const float *flat, size_t flat_offset, void *const *tensors,
                   const size_t *sizes, size_t count, float scale,
                   void *stream);
int sgb_unpack_f16_to_f32(const void *flat_f16, size_t flat_offset,
                          void *const *tensors, const size_t *sizes,
                          size_t count, float scale, void *stream);

/* ------------------------------------------------- sparsification kernels */
/* Workspace (256-byte aligned) for the two selectors below. */
size_t sgb_sparse_workspace_bytes(size_t n);
/* K of the top-K variant: (int)ceil(ratio * n) evaluated in fp32 exactly as
 * Communicator::topKSparsAllReduce does (src/io/communicator.cc:744). */
int sgb_topk_count(float ratio, size_t n);
/* Threshold selection with residual correction, one call for the sequence
 * add(acc) / backup / sparsabs / sub / sparsindex / removezeroidx /
 * removezeroval of Communicator::valSparsAllReduce (communicator.cc:626-680;
 * cuda::sparsabs, sparsindex, removezeroidx, removezeroval,
 * math_kernel.h:180-190):  s = g + acc; kept = |s| >= thr ? s : 0;
 * acc = s - kept; payload = (i+1, kept) for kept != 0 in ascending i.
 * acc may be NULL (no correction).  *nnz_dev (device) receives the count.
 * idx_out / val_out need room for n entries.  n <= 2^31-1. */
int sgb_sparse_threshold_f32(const float *g, float *acc, size_t n, float thr,
                             int32_t *idx_out, float *val_out,
                             int32_t *nnz_dev, void *ws, size_t ws_bytes,
                             void *stream);
/* Top-K selection with residual correction; replaces generateindex +
 * sortbykey (thrust::sort_by_key of all n pairs) + the cusparseSaxpyi
 * residual update of Communicator::topKSparsAllReduce (communicator.cc:
 * 721-765; math_kernel.h:184,190) by a 3-pass radix select.  s = g + acc is
 * formed once and kept in acc itself (sum_scratch is unused and may be NULL;
 * the argument remains for ABI stability).  The k entries with the largest key
 * are written in ascending index order, ties broken by lower index;
 * acc = s with the selected entries zeroed.
 * mode 0: key = |s|.  mode 1: key = |(int)s|, which is what the reference's
 * comparator evaluates (math_kernel.cu:715-721 truncates both operands to int).
 */
int sgb_sparse_topk_f32(const float *g, float *acc, float *sum_scratch,
                        size_t n, size_t k, int mode, int32_t *idx_out,
                        float *val_out, void *ws, size_t ws_bytes,
                        void *stream);
/* dst[idx[j]-1] += val[j] for j < count, or for j < min(*count_dev, count)
 * when count_dev is not NULL (count is then the capacity of idx / val);
 * idx 0 = padding, skipped.  Replaces cusparseSaxpyi with
 * CUSPARSE_INDEX_BASE_ONE (communicator.cc:715-717, 753-756, 803-805; the
 * routine no longer exists in CUDA 12).  n = length of dst. */
int sgb_scatter_add_f32(const int32_t *idx, const float *val, size_t count,
                        const int32_t *count_dev, float *dst, size_t n,
                        void *stream);

/* ------------------------------------------------------------ communicator */
/* Opaque handle standing in for class singa::Communicator
 * (include/singa/io/communicator.h:76-156, src/io/communicator.cc).  One per
 * process / GPU; creation binds to the CURRENT device, initialises the NCCL
 * communicator (ncclCommInitRank, communicator.cc:105-107), allocates the
 * two staging buffers of max_elems floats and three non-blocking side
 * streams (the reference takes them from Context: s, c1, c2,
 * src/core/device/cuda_gpu.cc:76-80).  Half and sparse buffers are allocated
 * at first use, as halfInit / sparsInit do (communicator.cc:114-139). */
typedef struct sgb_comm sgb_comm;
int sgb_last_nccl_error(void);
/* NcclIdHolder (communicator.cc:49-51): id_out receives
 * sgb_comm_unique_id_bytes() bytes to be shipped to every rank by the host. */
int sgb_comm_unique_id_bytes(void);
int sgb_comm_get_unique_id(void *id_out);
int sgb_comm_create(sgb_comm **out, int rank, int world, const void *unique_id,
                    size_t max_elems);
/* As sgb_comm_create, with NCCL's per-communicator limits on the number of
 * CTAs its kernels may use (ncclConfig_t minCTAs / maxCTAs; 0 = NCCL's
 * default): the collectives share the SMs with the backward kernels. */
int sgb_comm_create_ex(sgb_comm **out, int rank, int world,
                       const void *unique_id, size_t max_elems, int min_ctas,
                       int max_ctas);
/* Registers a caller-owned device buffer that will be reduced in place (a
 * gradient arena) with NCCL (ncclCommRegister), so that collectives on it can
 * use the registered-buffer protocols.  Deregistered by sgb_comm_destroy; the
 * buffer must outlive the communicator. */
int sgb_comm_register(sgb_comm *c, void *buffer, size_t bytes);
/* Makes the communicator issue its work on three CALLER-OWNED streams instead
 * of the ones it created: the reference's communicator takes s, c1 and c2 from
 * the device Context (src/core/device/cuda_gpu.cc:76-80), and its per-operation
 * time profiling records events on exactly those streams.  The three streams
 * must be distinct and must outlive the communicator; SGB_ERR_STATE while work
 * staged or enqueued since the last sgb_comm_wait is pending. */
int sgb_comm_use_streams(sgb_comm *c, void *s, void *c1, void *c2);
int sgb_comm_destroy(sgb_comm *c);
int sgb_comm_rank(const sgb_comm *c);
int sgb_comm_world_size(const sgb_comm *c);
size_t sgb_comm_staged_elems(const sgb_comm *c);
/* The three side streams (Context::s, c1, c2 of src/core/device/cuda_gpu.cc:
 * 76-80), for callers that profile or order against them: which = 0 (s, NCCL),
 * 1 (c1, pre-processing), 2 (c2, post-processing). */
void *sgb_comm_stream(const sgb_comm *c, int which);
/* The side stream on which the result of the most recent synch / flush /
 * sparsification call can be consumed (e.g. by an optimizer update enqueued
 * right behind it) without waiting for the rest of the backward pass:
 * c2 for in-place, fp16 and sparse results, c1 for an unpacked fp32 bucket.
 * Work put there is joined to the compute stream by the next sgb_comm_wait. */
void *sgb_comm_result_stream(const sgb_comm *c);
/* The communicator's cross-stream ordering rules as a pure host function (no
 * GPU needed): given the state {dirty_s, dirty_c1, dirty_c2, c2_reads_recv}
 * and a call kind (0 synch, 1 flush in place, 2 flush packed, 3 flush half,
 * 4 synch half, 5 sparsification, 6 stage copy, 7 wait) it updates the state
 * and returns the edge masks recorded before the pre-processing kernel,
 * before the collective, behind it, and behind the post-processing kernel
 * (bits: 1 compute->c1, 2 compute->s, 4 c1->s, 8 c2(done)->s, 16 s->c1,
 * 32 s->c2, 64 s->compute, 128 c1->compute, 256 c2->compute, 512 mark c2
 * done).  The communicator emits exactly these edges; the reference records
 * its compute-stream event before every stage and flush
 * (src/io/communicator.cc:227-233, 255-271, 313-319). */
int sgb_comm_order_plan(unsigned char *state4, int call, unsigned *edges4,
                        int *result_stream);
/* Per-phase device timing, the counterpart of the reference's time profiling
 * that brackets a "Dist_s_*" / "Dist_c1_*" / "Dist_c2_*" operation with events
 * on the stream its name selects (src/core/device/cuda_gpu.cc:128-169).
 * begin: records the origin on the compute stream and switches timing on;
 * every phase of every communicator call is then bracketed on its own side
 * stream under the reference's operation name (also emitted as NVTX ranges,
 * always).  range: brackets caller work on side stream `which` (begin != 0
 * opens, 0 closes the range opened last).  end: synchronises the device,
 * copies up to `capacity` rows (name, start and end in ms since the origin)
 * and switches timing off; *count receives the number of recorded phases.
 * Not usable while a stream is being captured (phases are then not timed). */
int sgb_comm_profile_begin(sgb_comm *c, void *compute_stream);
int sgb_comm_profile_range(sgb_comm *c, const char *name, int which, int begin);
/* A named point in time on any stream (start == end in the rows). */
int sgb_comm_profile_mark(sgb_comm *c, const char *name, void *stream);
int sgb_comm_profile_end(sgb_comm *c, char *names, size_t name_stride,
                         float *start_ms, float *end_ms, size_t capacity,
                         size_t *count);
/* 1 (default): top-K key as the reference's comparator computes it;
 * 0: key = |value|. */
int sgb_comm_set_topk_mode(sgb_comm *c, int mode);
/* Communicator::wait (communicator.cc:169-186): the compute stream waits for
 * the three side streams. */
int sgb_comm_wait(sgb_comm *c, void *compute_stream);
/* Communicator::synch (communicator.cc:304-328): in-place all-reduce(sum) on
 * stream s after the compute stream's work so far. */
int sgb_comm_synch(sgb_comm *c, void *data, size_t n, int is_half,
                   void *compute_stream);
/* Communicator::fusedSynch(t, send) (communicator.cc:212-302).  send == 0:
 * append the tensors to the bucket.  send != 0: all-reduce everything staged,
 * then scatter the result back into `tensors` (the full list staged since the
 * last flush, in staging order).  Staging is deferred: a stage call records
 * pointers and reserves space, and the bytes are gathered by one multi-tensor
 * pack launch at flush time, so a staged tensor must stay allocated and
 * unchanged until the flush (it has to: the flush writes the result into it).
 * When the staged tensors are exactly contiguous in memory (gradients kept in
 * one arena) and the flush list equals the staged list, the bucket is reduced
 * in place and no pack / unpack pass runs.  tensors / sizes are HOST arrays.
 * SGB_ERR_CAPACITY if the bucket would overflow. */
int sgb_comm_fused_synch(sgb_comm *c, void *const *tensors, const size_t *sizes,
                         size_t count, int is_half, int send,
                         void *compute_stream);
/* Communicator::synchHalf / fusedSynchHalf (communicator.cc:330-467): fp32
 * gradients are rounded to fp16, summed in fp16, widened back. */
int sgb_comm_synch_half(sgb_comm *c, float *data, size_t n,
                        void *compute_stream);
int sgb_comm_fused_synch_half(sgb_comm *c, void *const *tensors,
                              const size_t *sizes, size_t count, int send,
                              void *compute_stream);
/* Communicator::sparsification / fusedSparsification (communicator.cc:
 * 469-617) -> valSparsAllReduce / topKSparsAllReduce (:619-807).  count == 1
 * is the single-tensor form.  accumulation (device, total size) may be NULL.
 * topk == 0: spars is the magnitude threshold; the call blocks the host until
 * the per-rank counts have arrived (as the reference does).  topk != 0: spars
 * is the fraction of elements sent; fully asynchronous. */
int sgb_comm_sparsification(sgb_comm *c, void *const *tensors,
                            const size_t *sizes, size_t count,
                            float *accumulation, float spars, int topk,
                            void *compute_stream);
/* Threshold sparsification with a fixed exchange size: every rank sends
 * exactly `capacity` (index, value) slots, the true counts travel on the
 * device, and the host never waits for a count - so the call can sit inside a
 * captured graph (the reference, communicator.cc:657-669, reads the counts
 * back to size its all-gather).  Equal to sgb_comm_sparsification(topk = 0)
 * while a rank selects at most `capacity` entries.  Entries beyond that (in
 * index order) are not sent: with a residual buffer they stay in it and go out
 * with a later call; without one they are lost.  sgb_comm_sparse_dropped
 * returns how many entries this rank has held back so far (synchronises).
 * capacity <= the communicator's buffer size, else SGB_ERR_CAPACITY. */
int sgb_comm_sparsification_bounded(sgb_comm *c, void *const *tensors,
                                    const size_t *sizes, size_t count,
                                    float *accumulation, float threshold,
                                    size_t capacity, void *compute_stream);
int sgb_comm_sparse_dropped(sgb_comm *c, unsigned long long *dropped);


#ifdef __cplusplus
}
#endif
#endif /* SGB_H_ */
