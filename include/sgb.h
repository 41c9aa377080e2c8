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

const char *sgb_status_string(int status);
int sgb_last_cuda_error(void); /* last cudaError_t recorded by this library */
int sgb_version(void);

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

/* Strided gather out[i] = in[offset(i)] over an nDim-dimensional shape/stride
 * (element strides; 0 = broadcast).  Replaces cuda::traverse_unary_transform
 * (math_kernel.h:95-100) behind Transform<T, lang::Cuda>
 * (tensor_math_cuda.h:238-298).  shape/stride are HOST arrays, nDim <= 8:
 * they travel as kernel arguments, so no host-to-device copy is issued. */
int sgb_strided_copy_f32(const float *in, float *out, size_t n, int nDim,
                         const int *shape_host, const int *stride_host,
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

#ifdef __cplusplus
}
#endif
#endif /* SGB_H_ */
