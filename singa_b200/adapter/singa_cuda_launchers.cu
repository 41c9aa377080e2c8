// Source-compatible stand-in for SINGA's CUDA launcher layer, `namespace
// singa::cuda` (declared in src/core/tensor/math_kernel.h:41-193, defined in
// src/core/tensor/math_kernel.cu).  Every launcher keeps its exact C++
// signature - so tensor_math_cuda.h and communicator.cc link against this file
// instead of math_kernel.cu without an edit - and forwards to the C ABI of
// libsgb.so.  A non-zero status aborts, which is the reference's own error
// convention for this layer (CHECK / LOG(FATAL)).
//
// Built as libsgb_singa.so next to libsgb.so.  The mangled names exported here
// are compared with those of the reference's compiled math_kernel.cu, and the
// results of both are compared bit for bit, in the GPU tests.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "sgb.h"

namespace singa {
namespace cuda {

namespace {
inline void must(int status, const char* launcher) {
  if (status != SGB_OK) {
    std::fprintf(stderr, "singa::cuda::%s failed: %s (cuda error %d)\n", launcher,
                 sgb_status_string(status), sgb_last_cuda_error());
    std::abort();
  }
}
}  // namespace

#define SGB_F32_UNARY(NAME, OP)                                              \
  void NAME(const size_t n, const float* in, float* out, cudaStream_t s) {   \
    must(sgb_unary_f32(OP, in, out, n, s), #NAME);                           \
  }
#define SGB_F32_PAIR(NAME, OP)                                                                 \
  void NAME(const size_t n, const float* in1, const float* in2, float* out, cudaStream_t s) {  \
    must(sgb_binary_f32(OP, in1, in2, out, n, s), #NAME);                                      \
  }
#define SGB_F16_PAIR(NAME, OP)                                                                    \
  void NAME(const size_t n, const __half* in1, const __half* in2, __half* out, cudaStream_t s) {  \
    must(sgb_binary_f16(OP, in1, in2, out, n, s), #NAME);                                         \
  }
#define SGB_F32_WITH_SCALAR(NAME, OP)                                                       \
  void NAME(const size_t n, const float* in, const float x, float* out, cudaStream_t s) {   \
    must(sgb_scalar_f32(OP, in, x, out, n, s), #NAME);                                      \
  }
#define SGB_F32_SCALAR_FIRST(NAME, OP)                                                      \
  void NAME(const size_t n, const float x, const float* in, float* out, cudaStream_t s) {   \
    must(sgb_scalar_f32(OP, in, x, out, n, s), #NAME);                                      \
  }

// ---- no input
void set(const size_t n, const float v, float* out, cudaStream_t s) {
  must(sgb_set_f32(v, out, n, s), "set");
}

// ---- one input
SGB_F32_UNARY(abs, SGB_ABS)
SGB_F32_UNARY(sign, SGB_SIGN)
SGB_F32_UNARY(exp, SGB_EXP)
SGB_F32_UNARY(erf, SGB_ERF)
SGB_F32_UNARY(ceil2, SGB_CEIL)
SGB_F32_UNARY(floor, SGB_FLOOR)
SGB_F32_UNARY(round, SGB_ROUND)
SGB_F32_UNARY(rounde, SGB_ROUNDE)
SGB_F32_UNARY(log, SGB_LOG)
SGB_F32_UNARY(sqrt, SGB_SQRT)
SGB_F32_UNARY(square, SGB_SQUARE)
SGB_F32_UNARY(cos, SGB_COS)
SGB_F32_UNARY(cosh, SGB_COSH)
SGB_F32_UNARY(acos, SGB_ACOS)
SGB_F32_UNARY(acosh, SGB_ACOSH)
SGB_F32_UNARY(sin, SGB_SIN)
SGB_F32_UNARY(sinh, SGB_SINH)
SGB_F32_UNARY(asin, SGB_ASIN)
SGB_F32_UNARY(asinh, SGB_ASINH)
SGB_F32_UNARY(tan, SGB_TAN)
SGB_F32_UNARY(tanh, SGB_TANH)
SGB_F32_UNARY(atan, SGB_ATAN)
SGB_F32_UNARY(atanh, SGB_ATANH)
SGB_F32_UNARY(sigmoid, SGB_SIGMOID)
SGB_F32_UNARY(softplus, SGB_SOFTPLUS)
SGB_F32_UNARY(softsign, SGB_SOFTSIGN)

void relu(const size_t n, const float* in, float* out, cudaStream_t s) {
  must(sgb_relu_f32(in, out, n, s), "relu");
}
void relu(const size_t n, const __half* in, __half* out, cudaStream_t s) {
  must(sgb_relu_f16(in, out, n, s), "relu(half)");
}
void cast_float_2_int(const size_t n, const float* src, int* dst, cudaStream_t s) {
  must(sgb_cast_f32_i32(src, dst, n, s), "cast_float_2_int");
}
void cast_int_2_float(const size_t n, const int* src, float* dst, cudaStream_t s) {
  must(sgb_cast_i32_f32(src, dst, n, s), "cast_int_2_float");
}
void clamp(const size_t n, const float low, const float high, const float* in, float* out,
           cudaStream_t s) {
  must(sgb_clamp_f32(low, high, in, out, n, s), "clamp");
}
void float2half(const size_t n, const float* in, __half* out, cudaStream_t s) {
  must(sgb_cast_f32_f16(in, out, n, s), "float2half");
}
void half2float(const size_t n, const __half* in, float* out, cudaStream_t s) {
  must(sgb_cast_f16_f32(in, out, n, s), "half2float");
}

// ---- tensor (op) scalar
SGB_F32_WITH_SCALAR(pow, SGB_S_POW)
SGB_F32_WITH_SCALAR(add, SGB_S_ADD)
SGB_F32_WITH_SCALAR(mult, SGB_S_MUL)
SGB_F32_WITH_SCALAR(gt, SGB_S_GT)
SGB_F32_WITH_SCALAR(ge, SGB_S_GE)
SGB_F32_WITH_SCALAR(eq, SGB_S_EQ)
SGB_F32_WITH_SCALAR(lt, SGB_S_LT)
SGB_F32_WITH_SCALAR(le, SGB_S_LE)
SGB_F32_SCALAR_FIRST(div, SGB_S_RDIV)
SGB_F32_SCALAR_FIRST(threshold, SGB_S_THRESHOLD)
void mult(const size_t n, const __half* in, const __half x, __half* out, cudaStream_t s) {
  // the scalar is a half already: widening it and narrowing it again is exact
  must(sgb_scalar_mul_f16(in, __half2float(x), out, n, s), "mult(half, scalar)");
}

// ---- strided / broadcast gather; shape and stride are DEVICE arrays here
void traverse_unary_transform(const size_t n, size_t nDim, const float* in, const int* shape,
                              const int* stride, float* out, cudaStream_t s) {
  must(sgb_strided_copy_dev_f32(in, out, n, static_cast<int>(nDim), shape, stride, s),
       "traverse_unary_transform");
}
void traverse_unary_transform(const size_t n, size_t nDim, const __half* in, const int* shape,
                              const int* stride, __half* out, cudaStream_t s) {
  must(sgb_strided_copy_dev_f16(in, out, n, static_cast<int>(nDim), shape, stride, s),
       "traverse_unary_transform(half)");
}

// ---- tensor (op) tensor
void relubackward(const size_t num, const float* in1, const float* in2, float* out,
                  cudaStream_t s) {
  must(sgb_relu_backward_f32(in1, in2, out, num, s), "relubackward");
}
void relubackward(const size_t num, const __half* in1, const __half* in2, __half* out,
                  cudaStream_t s) {
  must(sgb_relu_backward_f16(in1, in2, out, num, s), "relubackward(half)");
}
SGB_F32_PAIR(gt, SGB_GT)
SGB_F32_PAIR(ge, SGB_GE)
SGB_F32_PAIR(eq, SGB_EQ)
SGB_F32_PAIR(lt, SGB_LT)
SGB_F32_PAIR(le, SGB_LE)
SGB_F32_PAIR(pow, SGB_POW)
SGB_F32_PAIR(add, SGB_ADD)
SGB_F32_PAIR(sub, SGB_SUB)
SGB_F32_PAIR(mult, SGB_MUL)
SGB_F32_PAIR(div, SGB_DIV)
SGB_F16_PAIR(pow, SGB_POW)
SGB_F16_PAIR(add, SGB_ADD)
SGB_F16_PAIR(sub, SGB_SUB)
SGB_F16_PAIR(mult, SGB_MUL)
SGB_F16_PAIR(div, SGB_DIV)

// ---- loss
void ComputeCrossEntropy(bool int_target, const size_t batchsize, const size_t dim, const float* p,
                         const int* t, float* loss, cudaStream_t stream) {
  must(sgb_cross_entropy_f32(int_target, batchsize, dim, p, t, loss, stream), "ComputeCrossEntropy");
}
void ComputeCrossEntropy(bool int_target, const size_t batchsize, const size_t dim, const __half* p,
                         const int* t, __half* loss, cudaStream_t stream) {
  must(sgb_cross_entropy_f16(int_target, batchsize, dim, p, t, loss, stream),
       "ComputeCrossEntropy(half)");
}
// The caller (tensor.cc:1717-1721) passes grad = a clone of p.  This form
// writes every element of grad from p, which gives the same tensor.
void SoftmaxCrossEntropyBwd(bool int_target, const size_t batchsize, const size_t dim,
                            const float* p, const int* t, float* grad, cudaStream_t stream) {
  must(sgb_softmax_cross_entropy_bwd_f32(int_target, batchsize, dim, p, t, grad, stream),
       "SoftmaxCrossEntropyBwd");
}
void SoftmaxCrossEntropyBwd(bool int_target, const size_t batchsize, const size_t dim,
                            const __half* p, const int* t, __half* grad, cudaStream_t stream) {
  must(sgb_softmax_cross_entropy_bwd_f16(int_target, batchsize, dim, p, t, grad, stream),
       "SoftmaxCrossEntropyBwd(half)");
}
void RowMax(const size_t nrow, const size_t ncol, const float* inPtr, float* outPtr,
            cudaStream_t stream) {
  must(sgb_row_max_f32(inPtr, outPtr, nrow, ncol, stream), "RowMax");
}

// ---- sparsification helpers of the communicator
void sparsabs(const size_t n, const float threshold, const float* in, float* out, cudaStream_t s) {
  must(sgb_sparsabs_f32(threshold, in, out, n, s), "sparsabs");
}
void sparsindex(const size_t n, const float* in, int* out, cudaStream_t s) {
  must(sgb_sparsindex_f32(in, out, n, s), "sparsindex");
}
void generateindex(const size_t n, int* out, cudaStream_t s) {
  must(sgb_generateindex_i32(out, n, s), "generateindex");
}
// removezeroval / removezeroidx / sortbykey (Thrust compaction and a full sort
// of value-index pairs) are not provided: their only caller is the
// communicator, whose replacement selects and compacts in sgb_sparse_*.

}  // namespace cuda
}  // namespace singa
