// Replacement for apache/singa's src/core/tensor/tensor_math_cuda.h: every
// `template <> void Op<DType, lang::Cuda>(..., Context* ctx)` specialisation
// that singa::Tensor math dispatches to on a CUDA device (the generic
// templates are declared in src/core/tensor/tensor_math.h:86-485), implemented
// over the C ABI of libsgb.so (include/sgb.h) - hand-written sm_100a kernels -
// instead of the one-element-per-thread launchers of math_kernel.cu, cuDNN's
// SetTensor / TransformTensor / OpTensor / Softmax / ReduceTensor calls and the
// cuBLAS level-1 routines.  src/core/tensor/tensor.cc includes the back-end
// headers exactly once (tensor.cc:22-25), so building that file with this
// header in place of the reference's (same include guard) switches the whole
// Tensor class over; nothing else in libsinga changes.
//
// What stays on the vendor libraries, as in the reference, because it is not
// part of the backward / gradient-synchronisation path: GEMV / GEMM /
// GEMMBatched (cuBLAS), the random generators (cuRAND) and SoftMaxBackward
// (cuDNN; the training path uses SoftmaxCrossEntropyBwd instead).
//
// Conventions: kernels run on ctx->stream; a non-zero status of the C ABI is
// fatal (LOG(FATAL)), like check_cudnn / CUBLAS_CHECK in the reference;
// temporaries are singa Tensors on the input's device, so they come from the
// device's memory pool and follow its release rule.
#ifndef SINGA_CORE_TENSOR_TENSOR_MATH_CUDA_H_
#define SINGA_CORE_TENSOR_TENSOR_MATH_CUDA_H_
#include "singa/singa_config.h"
#ifdef USE_CUDA
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cudnn.h>
#include <curand.h>

#include <vector>

#include "./tensor_math.h"
#include "sgb.h"
#include "singa/core/common.h"
#include "singa/core/tensor.h"
#include "singa/utils/cuda_utils.h"

namespace singa {
namespace sgb_backend {

inline void check(int status, const char* what) {
  if (status == SGB_OK) return;
  if (status == SGB_ERR_CUDA)
    LOG(FATAL) << what << ": " << sgb_status_string(status) << ": "
               << cudaGetErrorString(static_cast<cudaError_t>(sgb_last_cuda_error()));
  LOG(FATAL) << what << ": " << sgb_status_string(status) << " (status " << status << ")";
}
// The library reports launch errors through the runtime's per-thread last-error
// slot.  An error parked there by an earlier unchecked call of another library
// (SINGA itself checks no launches) is dropped first, so that it is not taken
// for this call's; sticky errors survive the read and are still reported.
#define SGB_CALL(call)                               \
  do {                                               \
    (void)cudaGetLastError();                        \
    ::singa::sgb_backend::check((call), #call);      \
  } while (0)
inline void check_cudnn_status(cudnnStatus_t status, const char* what) {
  if (status != CUDNN_STATUS_SUCCESS) LOG(FATAL) << what << ": " << cudnnGetErrorString(status);
}
#define SGB_CUDNN(call) ::singa::sgb_backend::check_cudnn_status((call), #call)

template <typename T>
inline const T* rd(const Tensor& t) {
  return static_cast<const T*>(t.block()->data());
}
template <typename T>
inline T* wr(Tensor* t) {
  return static_cast<T*>(t->block()->mutable_data());
}

// Contiguous copy of a strided / broadcast / transposed view: one gather
// kernel with shape and strides passed as kernel arguments (no descriptor, no
// host-to-device copy of the index tables).
template <typename T>
inline void gather(const Tensor& in, void* out, size_t n, Context* ctx) {
  const int nd = static_cast<int>(in.nDim());
  CHECK_LE(nd, 8) << "views of more than 8 dimensions are not supported";
  std::vector<int> shape(in.shape().begin(), in.shape().end());
  std::vector<int> stride(in.stride().begin(), in.stride().end());
  if (sizeof(T) == 4)
    SGB_CALL(sgb_strided_copy_f32(rd<float>(in), static_cast<float*>(out), n, nd, shape.data(), stride.data(),
                                  ctx->stream));
  else
    SGB_CALL(sgb_strided_copy_f16(in.block()->data(), out, n, nd, shape.data(), stride.data(), ctx->stream));
}

// The operand of an elementwise op as a dense array in the output's layout:
// the tensor's own memory when it already is, else a gathered copy held in
// `tmp`.
template <typename T>
inline const T* dense(const Tensor& in, const Tensor& like, Tensor* tmp, Context* ctx) {
  if (!in.broadcasted() && !in.transpose() && in.stride() == like.stride()) return rd<T>(in);
  *tmp = Tensor(in.shape(), in.device(), in.data_type());
  gather<T>(in, tmp->block()->mutable_data(), Product(in.shape()), ctx);
  return rd<T>(*tmp);
}

// True when the tensor's elements lie in memory in row-major order of its shape.
inline bool row_major(const Tensor& t) { return !t.transpose() && !t.broadcasted(); }

// out = f(in) for a one-input kernel: directly when the layouts agree;
// otherwise the input view is first gathered into a dense array and the
// kernel runs in place on it.  The dense array is `out` itself when `out` is
// row-major; when `out` is a transposed view (the reference writes it through
// a strided output descriptor) it is a temporary that is scattered into `out`.
template <typename Launch>
inline void unary_f32(const Tensor& in, Tensor* out, Context* ctx, Launch launch) {
  float* o = wr<float>(out);
  const size_t n = in.Size();
  if (in.stride() == out->stride()) {
    launch(rd<float>(in), o, n);
  } else if (row_major(*out)) {
    gather<float>(in, o, n, ctx);
    launch(o, o, n);
  } else {
    Tensor tmp(in.shape(), in.device(), kFloat32);
    float* d = wr<float>(&tmp);
    if (row_major(in)) {
      launch(rd<float>(in), d, n);
    } else {
      gather<float>(in, d, n, ctx);
      launch(d, d, n);
    }
    const int nd = static_cast<int>(out->nDim());
    CHECK_LE(nd, 8) << "views of more than 8 dimensions are not supported";
    std::vector<int> shape(out->shape().begin(), out->shape().end());
    std::vector<int> stride(out->stride().begin(), out->stride().end());
    SGB_CALL(sgb_strided_scatter_f32(d, o, n, nd, shape.data(), stride.data(), ctx->stream));
  }
}

template <typename T>
inline void binary(int op, const Tensor& a, const Tensor& b, Tensor* out, Context* ctx) {
  Tensor ta, tb;
  // the two operands only need to agree with EACH OTHER (the result is written
  // densely); an operand that is a plain dense array is used where it lies
  const Tensor& like = (!a.broadcasted() && !a.transpose()) ? a : b;
  const T* pa = dense<T>(a, like, &ta, ctx);
  const T* pb = dense<T>(b, like, &tb, ctx);
  if (sizeof(T) == 4)
    SGB_CALL(sgb_binary_f32(op, reinterpret_cast<const float*>(pa), reinterpret_cast<const float*>(pb),
                            wr<float>(out), out->Size(), ctx->stream));
  else
    SGB_CALL(sgb_binary_f16(op, pa, pb, out->block()->mutable_data(), out->Size(), ctx->stream));
}

// A one-element (or small) device scratch from the tensor's memory pool.
inline Tensor scratch_bytes(const Tensor& like, size_t bytes) {
  return Tensor(Shape{(bytes + 3) / 4 + 1}, like.device(), kFloat32);
}

}  // namespace sgb_backend

// ------------------------------------------------------------------ casts
template <>
void CastCopy<float, int, lang::Cuda>(const Tensor* src, Tensor* dst, Context* ctx) {
  SGB_CALL(sgb_cast_f32_i32(sgb_backend::rd<float>(*src), sgb_backend::wr<int32_t>(dst), dst->Size(), ctx->stream));
}
template <>
void CastCopy<int, float, lang::Cuda>(const Tensor* src, Tensor* dst, Context* ctx) {
  SGB_CALL(sgb_cast_i32_f32(sgb_backend::rd<int32_t>(*src), sgb_backend::wr<float>(dst), dst->Size(), ctx->stream));
}
template <>
void CastCopy<float, half_float::half, lang::Cuda>(const Tensor* src, Tensor* dst, Context* ctx) {
  SGB_CALL(sgb_cast_f32_f16(sgb_backend::rd<float>(*src), dst->block()->mutable_data(), dst->Size(), ctx->stream));
}
template <>
void CastCopy<half_float::half, float, lang::Cuda>(const Tensor* src, Tensor* dst, Context* ctx) {
  SGB_CALL(sgb_cast_f16_f32(src->block()->data(), sgb_backend::wr<float>(dst), dst->Size(), ctx->stream));
}

// ------------------------------------------------------------------- fill
template <>
void Set<float, lang::Cuda>(const float x, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_set_f32(x, sgb_backend::wr<float>(out), out->Size(), ctx->stream));
}
template <>
void Set<half_float::half, lang::Cuda>(const half_float::half x, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_set_f16(static_cast<float>(x), out->block()->mutable_data(), out->Size(), ctx->stream));
}

// -------------------------------------------- strided view -> dense array
template <>
void Transform<float, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  sgb_backend::gather<float>(in, out->block()->mutable_data(), Product(out->shape()), ctx);
}
template <>
void Transform<half_float::half, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  sgb_backend::gather<__half>(in, out->block()->mutable_data(), Product(out->shape()), ctx);
}
template <>
void Transform<__half, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  sgb_backend::gather<__half>(in, out->block()->mutable_data(), Product(out->shape()), ctx);
}

// ------------------------------------------------ tensor (op) tensor
#define SGB_BINARY(Name, OP)                                                                              \
  template <>                                                                                             \
  void Name<float, lang::Cuda>(const Tensor& a, const Tensor& b, Tensor* out, Context* ctx) {             \
    sgb_backend::binary<float>(OP, a, b, out, ctx);                                                       \
  }                                                                                                       \
  template <>                                                                                             \
  void Name<half_float::half, lang::Cuda>(const Tensor& a, const Tensor& b, Tensor* out, Context* ctx) {  \
    sgb_backend::binary<__half>(OP, a, b, out, ctx);                                                      \
  }
SGB_BINARY(Add, SGB_ADD)
SGB_BINARY(Sub, SGB_SUB)
SGB_BINARY(EltwiseMult, SGB_MUL)
SGB_BINARY(Div, SGB_DIV)
SGB_BINARY(Pow, SGB_POW)
#undef SGB_BINARY

// comparisons of two tensors: evaluated on the operands themselves (the
// reference subtracts first and compares the difference with zero, which
// gives the same 1.0 / 0.0 wherever the difference is representable)
#define SGB_COMPARE2(Name, OP)                                                                  \
  template <>                                                                                   \
  void Name<float, lang::Cuda>(const Tensor& a, const Tensor& b, Tensor* out, Context* ctx) {   \
    sgb_backend::binary<float>(SGB_SUB, a, b, out, ctx);                                        \
    float* o = sgb_backend::wr<float>(out);                                                     \
    SGB_CALL(sgb_scalar_f32(OP, o, 0.0f, o, out->Size(), ctx->stream));                         \
  }
SGB_COMPARE2(GE, SGB_S_GE)
SGB_COMPARE2(GT, SGB_S_GT)
SGB_COMPARE2(LE, SGB_S_LE)
SGB_COMPARE2(LT, SGB_S_LT)
SGB_COMPARE2(EQ, SGB_S_EQ)
#undef SGB_COMPARE2

// ------------------------------------------------ tensor (op) scalar
#define SGB_SCALAR(Name, OP)                                                                  \
  template <>                                                                                 \
  void Name<float, lang::Cuda>(const Tensor& in, const float x, Tensor* out, Context* ctx) {  \
    sgb_backend::unary_f32(in, out, ctx, [&](const float* i, float* o, size_t n) {            \
      SGB_CALL(sgb_scalar_f32(OP, i, x, o, n, ctx->stream));                                  \
    });                                                                                       \
  }
SGB_SCALAR(Add, SGB_S_ADD)
SGB_SCALAR(EltwiseMult, SGB_S_MUL)
SGB_SCALAR(Pow, SGB_S_POW)
SGB_SCALAR(GE, SGB_S_GE)
SGB_SCALAR(GT, SGB_S_GT)
SGB_SCALAR(LE, SGB_S_LE)
SGB_SCALAR(LT, SGB_S_LT)
SGB_SCALAR(EQ, SGB_S_EQ)
#undef SGB_SCALAR

template <>
void EltwiseMult<half_float::half, lang::Cuda>(const Tensor& in, const half_float::half x, Tensor* out,
                                               Context* ctx) {
  SGB_CALL(sgb_scalar_mul_f16(in.block()->data(), static_cast<float>(x), out->block()->mutable_data(), in.Size(),
                              ctx->stream));
}

/// out = x / in
template <>
void Div<float, lang::Cuda>(const float x, const Tensor& in, Tensor* out, Context* ctx) {
  sgb_backend::unary_f32(in, out, ctx, [&](const float* i, float* o, size_t n) {
    SGB_CALL(sgb_scalar_f32(SGB_S_RDIV, i, x, o, n, ctx->stream));
  });
}

template <>
void Clamp<float, lang::Cuda>(const float low, const float high, const Tensor& in, Tensor* out, Context* ctx) {
  sgb_backend::unary_f32(in, out, ctx, [&](const float* i, float* o, size_t n) {
    SGB_CALL(sgb_clamp_f32(low, high, i, o, n, ctx->stream));
  });
}

// ------------------------------------------------------------ one-input ops
#define SGB_UNARY(Name, OP)                                                           \
  template <>                                                                         \
  void Name<float, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {         \
    sgb_backend::unary_f32(in, out, ctx, [&](const float* i, float* o, size_t n) {    \
      SGB_CALL(sgb_unary_f32(OP, i, o, n, ctx->stream));                              \
    });                                                                               \
  }
SGB_UNARY(Abs, SGB_ABS)
SGB_UNARY(Sign, SGB_SIGN)
SGB_UNARY(Exp, SGB_EXP)
SGB_UNARY(Erf, SGB_ERF)
SGB_UNARY(Ceil, SGB_CEIL)
SGB_UNARY(Floor, SGB_FLOOR)
SGB_UNARY(Round, SGB_ROUND)
SGB_UNARY(RoundE, SGB_ROUNDE)
SGB_UNARY(Log, SGB_LOG)
SGB_UNARY(Sqrt, SGB_SQRT)
SGB_UNARY(Square, SGB_SQUARE)
SGB_UNARY(Cos, SGB_COS)
SGB_UNARY(Cosh, SGB_COSH)
SGB_UNARY(Acos, SGB_ACOS)
SGB_UNARY(Acosh, SGB_ACOSH)
SGB_UNARY(Sin, SGB_SIN)
SGB_UNARY(Sinh, SGB_SINH)
SGB_UNARY(Asin, SGB_ASIN)
SGB_UNARY(Asinh, SGB_ASINH)
SGB_UNARY(Tan, SGB_TAN)
SGB_UNARY(Tanh, SGB_TANH)
SGB_UNARY(Atan, SGB_ATAN)
SGB_UNARY(Atanh, SGB_ATANH)
SGB_UNARY(Sigmoid, SGB_SIGMOID)
SGB_UNARY(SoftPlus, SGB_SOFTPLUS)
SGB_UNARY(SoftSign, SGB_SOFTSIGN)
#undef SGB_UNARY

/// out = max(0, in)
template <>
void ReLU<float, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  sgb_backend::unary_f32(in, out, ctx, [&](const float* i, float* o, size_t n) {
    SGB_CALL(sgb_relu_f32(i, o, n, ctx->stream));
  });
}
template <>
void ReLU<half_float::half, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  void* o = out->block()->mutable_data();
  if (in.stride() == out->stride()) {
    SGB_CALL(sgb_relu_f16(in.block()->data(), o, in.Size(), ctx->stream));
  } else {
    sgb_backend::gather<__half>(in, o, in.Size(), ctx);
    SGB_CALL(sgb_relu_f16(o, o, in.Size(), ctx->stream));
  }
}
/// out = in2 > 0 ? in1 : 0 (in1 = upstream gradient, in2 = the ReLU's input)
template <>
void ReLUBackward<float, lang::Cuda>(const Tensor& in1, const Tensor& in2, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_relu_backward_f32(sgb_backend::rd<float>(in1), sgb_backend::rd<float>(in2), sgb_backend::wr<float>(out),
                                 in1.Size(), ctx->stream));
}
template <>
void ReLUBackward<half_float::half, lang::Cuda>(const Tensor& in1, const Tensor& in2, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_relu_backward_f16(in1.block()->data(), in2.block()->data(), out->block()->mutable_data(), in1.Size(),
                                 ctx->stream));
}

// ---------------------------------------------------------------- random
// The generators stay on cuRAND (ctx->curand_generator), as in the reference;
// the shaping passes behind them are kernels of this library.
template <>
void Bernoulli<float, lang::Cuda>(const float p, Tensor* out, Context* ctx) {
  float* o = sgb_backend::wr<float>(out);
  const size_t n = out->Size();
  CURAND_CHECK(curandGenerateUniform(ctx->curand_generator, o, n));
  SGB_CALL(sgb_scalar_f32(SGB_S_THRESHOLD, o, p, o, n, ctx->stream));
}
template <>
void Uniform<float, lang::Cuda>(const float low, const float high, Tensor* out, Context* ctx) {
  float* o = sgb_backend::wr<float>(out);
  const size_t n = out->Size();
  CURAND_CHECK(curandGenerateUniform(ctx->curand_generator, o, n));
  SGB_CALL(sgb_scalar_f32(SGB_S_MUL, o, high - low, o, n, ctx->stream));
  SGB_CALL(sgb_scalar_f32(SGB_S_ADD, o, low, o, n, ctx->stream));
}
template <>
void Gaussian<float, lang::Cuda>(const float mean, const float std, Tensor* out, Context* ctx) {
  const size_t n = out->Size();
  if (n % 2 == 0) {
    CURAND_CHECK(curandGenerateNormal(ctx->curand_generator, sgb_backend::wr<float>(out), n, mean, std));
    return;
  }
  // cuRAND's normal generator produces pairs: draw one more and drop it
  Tensor even(Shape{n + 1}, out->device());
  CURAND_CHECK(curandGenerateNormal(ctx->curand_generator, sgb_backend::wr<float>(&even), n + 1, mean, std));
  CopyDataToFrom(out, even, n, 0, 0);
}
template <>
void Uniform<half_float::half, lang::Cuda>(const half_float::half low, const half_float::half high, Tensor* out,
                                           Context* ctx) {
  Tensor wide(out->shape(), out->device(), kFloat32);
  Uniform<float, lang::Cuda>(static_cast<float>(low), static_cast<float>(high), &wide, ctx);
  CastCopy<float, half_float::half, lang::Cuda>(&wide, out, ctx);
}
template <>
void Gaussian<half_float::half, lang::Cuda>(const half_float::half mean, const half_float::half std, Tensor* out,
                                            Context* ctx) {
  Tensor wide(out->shape(), out->device(), kFloat32);
  Gaussian<float, lang::Cuda>(static_cast<float>(mean), static_cast<float>(std), &wide, ctx);
  CastCopy<float, half_float::half, lang::Cuda>(&wide, out, ctx);
}

// --------------------------------------------------------- BLAS level 1
// Reductions leave their result on the device; the forms that return a host
// scalar copy it back on ctx->stream and wait for that stream.
namespace sgb_backend {
template <typename R, typename Launch>
inline R reduce_to_host(const Tensor& in, Context* ctx, Launch launch) {
  const size_t ws_bytes = sgb_blas1_workspace_bytes(in.Size());
  Tensor ws = scratch_bytes(in, ws_bytes), result = scratch_bytes(in, sizeof(R));
  launch(wr<float>(&result), wr<float>(&ws), ws.Size() * sizeof(float));
  R host = R();
  CUDA_CHECK(cudaMemcpyAsync(&host, result.block()->data(), sizeof(R), cudaMemcpyDeviceToHost, ctx->stream));
  CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return host;
}
}  // namespace sgb_backend

template <>
void Amax<float, lang::Cuda>(const Tensor& in, size_t* out, Context* ctx) {
  *out = static_cast<size_t>(sgb_backend::reduce_to_host<int32_t>(in, ctx, [&](float* r, float* ws, size_t wb) {
    SGB_CALL(sgb_amax_f32(sgb_backend::rd<float>(in), reinterpret_cast<int32_t*>(r), in.Size(), ws, wb, ctx->stream));
  }));
}
template <>
void Amin<float, lang::Cuda>(const Tensor& in, size_t* out, Context* ctx) {
  *out = static_cast<size_t>(sgb_backend::reduce_to_host<int32_t>(in, ctx, [&](float* r, float* ws, size_t wb) {
    SGB_CALL(sgb_amin_f32(sgb_backend::rd<float>(in), reinterpret_cast<int32_t*>(r), in.Size(), ws, wb, ctx->stream));
  }));
}
template <>
void Asum<float, lang::Cuda>(const Tensor& in, float* out, Context* ctx) {
  *out = sgb_backend::reduce_to_host<float>(in, ctx, [&](float* r, float* ws, size_t wb) {
    SGB_CALL(sgb_asum_f32(sgb_backend::rd<float>(in), r, in.Size(), ws, wb, ctx->stream));
  });
}
template <>
void Nrm2<float, lang::Cuda>(const Tensor& in, float* out, Context* ctx) {
  *out = sgb_backend::reduce_to_host<float>(in, ctx, [&](float* r, float* ws, size_t wb) {
    SGB_CALL(sgb_nrm2_f32(sgb_backend::rd<float>(in), r, in.Size(), ws, wb, ctx->stream));
  });
}
template <>
void Dot<float, lang::Cuda>(const Tensor& in1, const Tensor& in2, float* out, Context* ctx) {
  *out = sgb_backend::reduce_to_host<float>(in1, ctx, [&](float* r, float* ws, size_t wb) {
    SGB_CALL(sgb_dot_f32(sgb_backend::rd<float>(in1), sgb_backend::rd<float>(in2), r, in1.Size(), ws, wb, ctx->stream));
  });
}
/// the result stays on the device (used by SumAll: no host round trip)
template <>
void Dot<float, lang::Cuda>(const Tensor& in1, const Tensor& in2, Tensor* out, Context* ctx) {
  const size_t wb = sgb_blas1_workspace_bytes(in1.Size());
  Tensor ws = sgb_backend::scratch_bytes(in1, wb);
  SGB_CALL(sgb_dot_f32(sgb_backend::rd<float>(in1), sgb_backend::rd<float>(in2), sgb_backend::wr<float>(out),
                       in1.Size(), sgb_backend::wr<float>(&ws), ws.Size() * sizeof(float), ctx->stream));
}
template <>
void Dot<half_float::half, lang::Cuda>(const Tensor& in1, const Tensor& in2, Tensor* out, Context* ctx) {
  // fp16 operands, fp32 accumulation, fp16 result: widen, reduce, narrow
  Tensor a = in1.AsType(kFloat32), b = in2.AsType(kFloat32), r(Shape{1}, in1.device(), kFloat32);
  Dot<float, lang::Cuda>(a, b, &r, ctx);
  CastCopy<float, half_float::half, lang::Cuda>(&r, out, ctx);
}

/// out += alpha * in
template <>
void Axpy<float, lang::Cuda>(const float alpha, const Tensor& in, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_axpy_f32(alpha, sgb_backend::rd<float>(in), sgb_backend::wr<float>(out), in.Size(), ctx->stream));
}
/// alpha is a one-element device tensor (the optimizer keeps its hyper-parameters on the device)
template <>
void Axpy<float, lang::Cuda>(const Tensor& alpha, const Tensor& in, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_axpy_dev_alpha_f32(sgb_backend::rd<float>(alpha), sgb_backend::rd<float>(in), sgb_backend::wr<float>(out),
                                  in.Size(), ctx->stream));
}
template <>
void Axpy<half_float::half, lang::Cuda>(const Tensor& alpha, const Tensor& in, Tensor* out, Context* ctx) {
  Tensor wide = alpha.AsType(kFloat32);
  SGB_CALL(sgb_axpy_dev_alpha_f16(sgb_backend::rd<float>(wide), in.block()->data(), out->block()->mutable_data(),
                                  in.Size(), ctx->stream));
}
template <>
void Axpy<half_float::half, lang::Cuda>(const half_float::half alpha, const Tensor& in, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_axpy_f16(static_cast<float>(alpha), in.block()->data(), out->block()->mutable_data(), in.Size(),
                        ctx->stream));
}
/// out *= x
template <>
void Scale<float, lang::Cuda>(const float x, Tensor* out, Context* ctx) {
  float* o = sgb_backend::wr<float>(out);
  SGB_CALL(sgb_scalar_f32(SGB_S_MUL, o, x, o, out->Size(), ctx->stream));
}
/// out = M diag(v) (side_right) or diag(v) M, M row-major
template <>
void DGMM<float, lang::Cuda>(const bool side_right, const Tensor& M, const Tensor& v, Tensor* out, Context* ctx) {
  SGB_CALL(sgb_dgmm_f32(side_right ? 1 : 0, sgb_backend::rd<float>(M), sgb_backend::rd<float>(v),
                        sgb_backend::wr<float>(out), M.shape(0), M.shape(1), ctx->stream));
}

// ------------------------------------------- contractions (cuBLAS, unchanged)
// Row-major operands are handed to the column-major library as their
// transposes: C = A B is computed as C^T = B^T A^T.
namespace sgb_backend {
struct MatDims {
  cublasOperation_t op_a, op_b;
  int rows_a, cols_a, cols_b, lda, ldb, ldc;
  MatDims(const Tensor& A, const Tensor& B) {
    const size_t nd = A.nDim();
    rows_a = static_cast<int>(A.shape(nd - 2));
    cols_a = static_cast<int>(A.shape(nd - 1));
    cols_b = static_cast<int>(B.shape(B.nDim() - 1));
    op_a = A.transpose() ? CUBLAS_OP_T : CUBLAS_OP_N;
    op_b = B.transpose() ? CUBLAS_OP_T : CUBLAS_OP_N;
    lda = A.transpose() ? rows_a : cols_a;
    ldb = B.transpose() ? cols_a : cols_b;
    ldc = cols_b;
  }
};
}  // namespace sgb_backend

template <>
void GEMM<float, lang::Cuda>(const float alpha, const Tensor& A, const Tensor& B, const float beta, Tensor* C,
                             Context* ctx) {
  const sgb_backend::MatDims d(A, B);
  CUBLAS_CHECK(cublasSgemm(ctx->cublas_handle, d.op_b, d.op_a, d.cols_b, d.rows_a, d.cols_a, &alpha,
                           sgb_backend::rd<float>(B), d.ldb, sgb_backend::rd<float>(A), d.lda, &beta,
                           sgb_backend::wr<float>(C), d.ldc));
}
template <>
void GEMM<half_float::half, lang::Cuda>(const half_float::half alpha, const Tensor& A, const Tensor& B,
                                        const half_float::half beta, Tensor* C, Context* ctx) {
  const sgb_backend::MatDims d(A, B);
  const __half a = __float2half(static_cast<float>(alpha)), b = __float2half(static_cast<float>(beta));
  CUBLAS_CHECK(cublasHgemm(ctx->cublas_handle, d.op_b, d.op_a, d.cols_b, d.rows_a, d.cols_a, &a,
                           sgb_backend::rd<__half>(B), d.ldb, sgb_backend::rd<__half>(A), d.lda, &b,
                           sgb_backend::wr<__half>(C), d.ldc));
}
template <>
void GEMMBatched<float, lang::Cuda>(const float alpha, const Tensor& A, const Tensor& B, const float beta,
                                    Tensor* C, Context* ctx) {
  const sgb_backend::MatDims d(A, B);
  size_t batch = A.shape(0);
  if (A.nDim() == 4u) batch *= A.shape(1);
  const long long stride_a = static_cast<long long>(d.rows_a) * d.cols_a;
  const long long stride_b = static_cast<long long>(d.cols_a) * d.cols_b;
  const long long stride_c = static_cast<long long>(d.rows_a) * d.cols_b;
  CUBLAS_CHECK(cublasSgemmStridedBatched(ctx->cublas_handle, d.op_b, d.op_a, d.cols_b, d.rows_a, d.cols_a, &alpha,
                                         sgb_backend::rd<float>(B), d.ldb, stride_b, sgb_backend::rd<float>(A), d.lda,
                                         stride_a, &beta, sgb_backend::wr<float>(C), d.ldc, stride_c,
                                         static_cast<int>(batch)));
}
/// out = alpha * A v + beta * out, A row-major m x n (or its transposed view)
template <>
void GEMV<float, lang::Cuda>(const float alpha, const Tensor& A, const Tensor& v, const float beta, Tensor* out,
                             Context* ctx) {
  const int m = static_cast<int>(A.shape(0)), n = static_cast<int>(A.shape(1));
  if (A.transpose())
    CUBLAS_CHECK(cublasSgemv(ctx->cublas_handle, CUBLAS_OP_N, m, n, &alpha, sgb_backend::rd<float>(A), m,
                             sgb_backend::rd<float>(v), 1, &beta, sgb_backend::wr<float>(out), 1));
  else
    CUBLAS_CHECK(cublasSgemv(ctx->cublas_handle, CUBLAS_OP_T, n, m, &alpha, sgb_backend::rd<float>(A), n,
                             sgb_backend::rd<float>(v), 1, &beta, sgb_backend::wr<float>(out), 1));
}
template <>
void GEMV<half_float::half, lang::Cuda>(const half_float::half alpha, const Tensor& A, const Tensor& v,
                                        const half_float::half beta, Tensor* out, Context* ctx) {
  Tensor wide_a = A.AsType(kFloat32), wide_v = v.AsType(kFloat32), wide_out(out->shape(), out->device(), kFloat32);
  GEMV<float, lang::Cuda>(static_cast<float>(alpha), wide_a, wide_v, static_cast<float>(beta), &wide_out, ctx);
  CastCopy<float, half_float::half, lang::Cuda>(&wide_out, out, ctx);
}

// ------------------------------------------------------ softmax / loss head
// Softmax over everything but the leading dimension, one instance per leading
// index (what the reference asks of cuDNN with SOFTMAX_ACCURATE / MODE_INSTANCE
// on an {N, C, 1, 1} view): rows = shape[0], columns = the rest.
namespace sgb_backend {
inline void softmax_extent(const Tensor& in, size_t* rows, size_t* cols) {
  *rows = in.nDim() ? in.shape(0) : 1;
  *cols = *rows ? in.Size() / *rows : 0;
}
}  // namespace sgb_backend

template <>
void SoftMax<float, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  size_t rows, cols;
  sgb_backend::softmax_extent(in, &rows, &cols);
  SGB_CALL(sgb_softmax_rows_f32(sgb_backend::rd<float>(in), sgb_backend::wr<float>(out), rows, cols, ctx->stream));
}
template <>
void SoftMax<half_float::half, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  size_t rows, cols;
  sgb_backend::softmax_extent(in, &rows, &cols);
  SGB_CALL(sgb_softmax_rows_f16(in.block()->data(), out->block()->mutable_data(), rows, cols, ctx->stream));
}
/// Gradient of a stand-alone softmax (not on the training path): cuDNN, as in the reference.
template <>
void SoftMaxBackward<float, lang::Cuda>(const Tensor& in, Tensor* out, const Tensor& fdout, Context* ctx) {
  size_t rows, cols;
  sgb_backend::softmax_extent(in, &rows, &cols);
  cudnnTensorDescriptor_t desc;
  SGB_CUDNN(cudnnCreateTensorDescriptor(&desc));
  SGB_CUDNN(cudnnSetTensor4dDescriptor(desc, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, static_cast<int>(rows),
                                         static_cast<int>(cols), 1, 1));
  const float one = 1.0f, zero = 0.0f;
  SGB_CUDNN(cudnnSoftmaxBackward(ctx->cudnn_handle, CUDNN_SOFTMAX_ACCURATE, CUDNN_SOFTMAX_MODE_INSTANCE, &one, desc,
                                   sgb_backend::rd<float>(fdout), desc, sgb_backend::rd<float>(in), &zero, desc,
                                   sgb_backend::wr<float>(out)));
  SGB_CUDNN(cudnnDestroyTensorDescriptor(desc));
}

template <>
void ComputeCrossEntropy<float, lang::Cuda>(bool int_target, const size_t batchsize, const size_t dim,
                                            const Tensor& p, const Tensor& t, Tensor* loss, Context* ctx) {
  SGB_CALL(sgb_cross_entropy_f32(int_target ? 1 : 0, batchsize, dim, sgb_backend::rd<float>(p),
                                 sgb_backend::rd<int32_t>(t), sgb_backend::wr<float>(loss), ctx->stream));
}
template <>
void ComputeCrossEntropy<half_float::half, lang::Cuda>(bool int_target, const size_t batchsize, const size_t dim,
                                                       const Tensor& p, const Tensor& t, Tensor* loss, Context* ctx) {
  SGB_CALL(sgb_cross_entropy_f16(int_target ? 1 : 0, batchsize, dim, p.block()->data(), sgb_backend::rd<int32_t>(t),
                                 loss->block()->mutable_data(), ctx->stream));
}
/// grad = p - onehot(t), written over p (the caller passes the same block for both)
template <>
void SoftmaxCrossEntropyBwd<float, lang::Cuda>(bool int_target, const size_t batchsize, const size_t dim,
                                               const Tensor& p, const Tensor& t, Tensor* grad, Context* ctx) {
  CHECK_EQ(p.block(), grad->block()) << "the gradient is computed in place over the probabilities";
  SGB_CALL(sgb_softmax_cross_entropy_bwd_f32(int_target ? 1 : 0, batchsize, dim, sgb_backend::rd<float>(p),
                                             sgb_backend::rd<int32_t>(t), sgb_backend::wr<float>(grad), ctx->stream));
}
template <>
void SoftmaxCrossEntropyBwd<half_float::half, lang::Cuda>(bool int_target, const size_t batchsize, const size_t dim,
                                                          const Tensor& p, const Tensor& t, Tensor* grad,
                                                          Context* ctx) {
  CHECK_EQ(p.block(), grad->block()) << "the gradient is computed in place over the probabilities";
  SGB_CALL(sgb_softmax_cross_entropy_bwd_f16(int_target ? 1 : 0, batchsize, dim, p.block()->data(),
                                             sgb_backend::rd<int32_t>(t), grad->block()->mutable_data(), ctx->stream));
}

// --------------------------------------------------------------- reductions
template <>
void RowMax<float, lang::Cuda>(const Tensor& in, Tensor* out, Context* ctx) {
  Tensor tmp;
  const float* m = sgb_backend::rd<float>(in);
  if (in.transpose()) {
    tmp = Tensor(in.shape(), in.device(), in.data_type());
    sgb_backend::gather<float>(in, tmp.block()->mutable_data(), in.Size(), ctx);
    m = sgb_backend::rd<float>(tmp);
  }
  SGB_CALL(sgb_row_max_f32(m, sgb_backend::wr<float>(out), in.shape(0), in.shape(1), ctx->stream));
}
/// Sum of all elements, returned on the host.
template <>
void Sum<float, lang::Cuda>(const Tensor& in, float* out, Context* ctx) {
  const size_t wb = sgb_sum_all_workspace_bytes(in.Size());
  Tensor ws = sgb_backend::scratch_bytes(in, wb), r(Shape{1}, in.device(), kFloat32);
  SGB_CALL(sgb_sum_all_f32(sgb_backend::rd<float>(in), sgb_backend::wr<float>(&r), in.Size(),
                           sgb_backend::wr<float>(&ws), ws.Size() * sizeof(float), ctx->stream));
  CUDA_CHECK(cudaMemcpyAsync(out, r.block()->data(), sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
}

#undef SGB_CALL
#undef SGB_CUDNN
}  // namespace singa
#endif  // USE_CUDA
#endif  // SINGA_CORE_TENSOR_TENSOR_MATH_CUDA_H_
