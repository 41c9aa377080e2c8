// extern "C" doors into an apache/singa core library built for CUDA
// (oracle/ref_cuda_build.py).  TEST INFRASTRUCTURE ONLY.  Everything here is
// written against the reference's PUBLIC C++ interface only - singa::Tensor
// and its free functions (include/singa/core/tensor.h), the operation handles
// and Gpu* functions (src/model/operation/batchnorm.h, pooling.h) and
// class Communicator (include/singa/io/communicator.h) - so the same file is
// compiled twice: once with the reference's own CUDA back end (the comparator)
// and once with this repository's replacement back end (tensor_math_cuda.h,
// operation and communicator adapters).  A test that drives both through these
// doors checks the replacement on the reference's own types.
//
// Tensors are created on one singa::CudaGPU device and referred to by opaque
// handles; functions that return a Tensor in the reference return a new
// handle (the caller frees it).
#include <cstring>
#include <memory>
#include <vector>

#include "singa/core/device.h"
#include "singa/core/tensor.h"
#include "singa/io/communicator.h"
#include "model/operation/batchnorm.h"
#include "model/operation/pooling.h"
#ifdef SGB_VARIANT
#include "model/operation/convolution.h"
#endif

using singa::Shape;
using singa::Tensor;

namespace {
std::shared_ptr<singa::Device> g_dev;

Tensor* own(const Tensor& t) { return new Tensor(t); }
Tensor& T(void* h) { return *static_cast<Tensor*>(h); }
}  // namespace

extern "C" {

int rs_init(int device_id) {
  if (!g_dev) g_dev = std::make_shared<singa::CudaGPU>(device_id);
  return 0;
}

void rs_sync() {
  if (g_dev) g_dev->Sync();
}

// dtype: 0 float32, 1 float16, 2 int32
void* rs_tensor_new(int ndim, const size_t* dims, int dtype) {
  Shape s(dims, dims + ndim);
  const singa::DataType dt = dtype == 1 ? singa::kFloat16 : (dtype == 2 ? singa::kInt : singa::kFloat32);
  Tensor* t = new Tensor(s, g_dev, dt);
  t->block()->mutable_data();   // allocate now: callers take the device pointer
  return t;
}
void rs_tensor_free(void* h) { delete static_cast<Tensor*>(h); }
void* rs_tensor_ptr(void* h) { return T(h).block()->mutable_data(); }
size_t rs_tensor_size(void* h) { return T(h).Size(); }
int rs_tensor_ndim(void* h) { return static_cast<int>(T(h).shape().size()); }
size_t rs_tensor_dim(void* h, int i) { return T(h).shape()[i]; }
void rs_tensor_from_host_f32(void* h, const float* src) { T(h).CopyDataFromHostPtr(src, T(h).Size()); }
void rs_tensor_from_host_i32(void* h, const int* src) { T(h).CopyDataFromHostPtr(src, T(h).Size()); }
void rs_tensor_to_host_f32(void* h, float* dst) {
  Tensor c = T(h).Clone(singa::defaultDevice);
  c.GetValue(dst, c.Size());
}
void rs_tensor_set(void* h, float v) { T(h).SetValue(v); }
// Fills the tensor from `bytes` bytes of device memory owned by someone else
// (a plain device-to-device copy on the default stream).
int rs_tensor_from_device(void* h, const void* src, size_t bytes) {
  return static_cast<int>(cudaMemcpy(T(h).block()->mutable_data(), src, bytes, cudaMemcpyDeviceToDevice));
}
int rs_tensor_to_device(void* h, void* dst, size_t bytes) {
  return static_cast<int>(cudaMemcpy(dst, T(h).block()->data(), bytes, cudaMemcpyDeviceToDevice));
}
void* rs_tensor_as_type(void* h, int dtype) {
  return own(T(h).AsType(dtype == 1 ? singa::kFloat16 : (dtype == 2 ? singa::kInt : singa::kFloat32)));
}

// ------------------------------------------------------------- tensor math
void* rs_relu(void* x) { return own(singa::ReLU(T(x))); }
void* rs_relu_backward(void* dy, void* x) { return own(singa::ReLUBackward(T(dy), T(x))); }
void* rs_add(void* a, void* b) { return own(T(a) + T(b)); }
void* rs_sub(void* a, void* b) { return own(T(a) - T(b)); }
void* rs_eltwise_mult(void* a, void* b) { return own(T(a) * T(b)); }
void* rs_div(void* a, void* b) { return own(T(a) / T(b)); }
void rs_add_inplace(void* a, void* b) { T(a) += T(b); }
void rs_mult_scalar_inplace(void* a, float c) { T(a) *= c; }
void rs_div_scalar_inplace(void* a, float c) { T(a) /= c; }
void* rs_sum_axis(void* a, int axis) { return own(singa::Sum(T(a), axis)); }
void* rs_sum_all(void* a) { return own(singa::SumAll(T(a))); }
void* rs_softmax(void* a) { return own(singa::SoftMax(T(a))); }
void* rs_cross_entropy_fwd(void* p, void* t) { return own(singa::CrossEntropyFwd(T(p), T(t))); }
void* rs_softmax_cross_entropy_bwd(void* p, void* t) { return own(singa::SoftmaxCrossEntropyBwd(T(p), T(t))); }
void rs_axpy(float alpha, void* x, void* y) { singa::Axpy(alpha, T(x), &T(y)); }
void* rs_mult(void* a, void* b) { return own(singa::Mult(T(a), T(b))); }
void* rs_transpose(void* a) { return own(singa::Transpose(T(a))); }
// unary ops by name index: 0 exp 1 log 2 sqrt 3 tanh 4 sigmoid 5 abs 6 sign 7 square 8 softplus 9 softsign
void* rs_unary(int op, void* a) {
  switch (op) {
    case 0: return own(singa::Exp(T(a)));
    case 1: return own(singa::Log(T(a)));
    case 2: return own(singa::Sqrt(T(a)));
    case 3: return own(singa::Tanh(T(a)));
    case 4: return own(singa::Sigmoid(T(a)));
    case 5: return own(singa::Abs(T(a)));
    case 6: return own(singa::Sign(T(a)));
    case 7: return own(singa::Square(T(a)));
    case 8: return own(singa::SoftPlus(T(a)));
    case 9: return own(singa::SoftSign(T(a)));
    default: return nullptr;
  }
}
// comparisons with a scalar: 0 LT 1 LE 2 GT 3 GE 4 EQ
void* rs_compare_scalar(int op, void* a, float c) {
  switch (op) {
    case 0: return own(T(a) < c);
    case 1: return own(T(a) <= c);
    case 2: return own(T(a) > c);
    case 3: return own(T(a) >= c);
    case 4: return own(T(a) == c);
    default: return nullptr;
  }
}
void rs_mult_column(void* v, void* m) { singa::MultColumn(T(v), &T(m)); }
void rs_mult_row(void* v, void* m) { singa::MultRow(T(v), &T(m)); }
void rs_add_row(void* v, void* m) { singa::AddRow(T(v), &T(m)); }
void* rs_row_max(void* a) { return own(singa::RowMax(T(a))); }
float rs_l2(void* a) { return T(a).L2(); }
float rs_l1(void* a) { return T(a).L1(); }

// The optimizer's call chain on one parameter (python/singa/opt.py:269-310).
void rs_sgd(void* param, void* grad, void* moment, float lr, float momentum, float weight_decay) {
  Tensor g = T(grad);
  if (weight_decay != 0.0f) singa::Axpy(weight_decay, T(param), &g);
  if (momentum != 0.0f) {
    T(moment) *= momentum;
    singa::Axpy(1.0f, g, &T(moment));
    g = T(moment);
  }
  singa::Axpy(-lr, g, &T(param));
}

// -------------------------------------------------------- operation handles
void* rs_bn_handle_new(float momentum, void* x) { return new singa::CudnnBatchNormHandle(momentum, T(x)); }
void rs_bn_handle_free(void* h) { delete static_cast<singa::CudnnBatchNormHandle*>(h); }
// out[0..2] = y, saved mean, saved inverse std
void rs_bn_forward_training(void* h, void* x, void* scale, void* bias, void* running_mean, void* running_var,
                            void** out) {
  const std::vector<Tensor> r = singa::GpuBatchNormForwardTraining(
      *static_cast<singa::CudnnBatchNormHandle*>(h), T(x), T(scale), T(bias), T(running_mean), T(running_var));
  for (int i = 0; i < 3; ++i) out[i] = own(r[i]);
}
// out[0..2] = dx, dscale, dbias
void rs_bn_backward(void* h, void* dy, void* x, void* scale, void* mean, void* var, void** out) {
  const std::vector<Tensor> r = singa::GpuBatchNormBackward(*static_cast<singa::CudnnBatchNormHandle*>(h), T(dy),
                                                            T(x), T(scale), T(mean), T(var));
  for (int i = 0; i < 3; ++i) out[i] = own(r[i]);
}
void* rs_pool_handle_new(void* x, int kh, int kw, int sh, int sw, int ph, int pw, int is_max) {
  return new singa::CudnnPoolingHandle(T(x), {kh, kw}, {sh, sw}, {ph, pw}, is_max != 0);
}
void rs_pool_handle_free(void* h) { delete static_cast<singa::CudnnPoolingHandle*>(h); }
void* rs_pool_forward(void* h, void* x) {
  return own(singa::GpuPoolingForward(*static_cast<singa::CudnnPoolingHandle*>(h), T(x)));
}
void* rs_pool_backward(void* h, void* dy, void* x, void* y) {
  return own(singa::GpuPoolingBackward(*static_cast<singa::CudnnPoolingHandle*>(h), T(dy), T(x), T(y)));
}

#ifdef SGB_VARIANT
// Bias gradient of a convolution.  Only in the build with this repository's
// back end: the reference's convolution.cc does not compile against cuDNN 9,
// so no handle can be constructed; the replacement never reads the handle, and
// a zeroed stand-in object is passed by reference.
void* rs_conv_bias_backward(void* dy, void* b) {
  alignas(16) static unsigned char storage[sizeof(singa::CudnnConvHandle)] = {};
  const singa::CudnnConvHandle& fake = *reinterpret_cast<const singa::CudnnConvHandle*>(storage);
  return own(singa::GpuConvBackwardb(T(dy), T(b), fake));
}
int rs_variant() { return 1; }
#else
int rs_variant() { return 0; }
#endif

// ------------------------------------------------------------- communicator
int rs_nccl_id_bytes() { return static_cast<int>(sizeof(ncclUniqueId)); }
void rs_nccl_id_new(void* out) {
  singa::NcclIdHolder holder;
  std::memcpy(out, &holder.id, sizeof(holder.id));
}
void* rs_comm_new(int local_rank, int world, const void* id, int buff_size) {
  singa::NcclIdHolder holder;
  std::memcpy(&holder.id, id, sizeof(holder.id));
  return new singa::Communicator(local_rank, world, holder, buff_size);
}
void rs_comm_free(void* c) { delete static_cast<singa::Communicator*>(c); }
int rs_comm_rank(void* c) { return static_cast<singa::Communicator*>(c)->global_rank; }
int rs_comm_world(void* c) { return static_cast<singa::Communicator*>(c)->world_size; }
void rs_comm_synch(void* c, void* t) { static_cast<singa::Communicator*>(c)->synch(T(t)); }
void rs_comm_synch_half(void* c, void* t) { static_cast<singa::Communicator*>(c)->synchHalf(T(t)); }
static std::vector<Tensor> list_of(void** ts, int n) {
  std::vector<Tensor> v;
  for (int i = 0; i < n; ++i) v.push_back(T(ts[i]));
  return v;
}
void rs_comm_fused_synch(void* c, void** ts, int n, int send) {
  std::vector<Tensor> v = list_of(ts, n);
  static_cast<singa::Communicator*>(c)->fusedSynch(v, send != 0);
}
void rs_comm_fused_synch_half(void* c, void** ts, int n, int send) {
  std::vector<Tensor> v = list_of(ts, n);
  static_cast<singa::Communicator*>(c)->fusedSynchHalf(v, send != 0);
}
// accumulation may be NULL.  Only top-K is exercised on the reference build:
// its threshold path reads a count from unspecified memory.
void rs_comm_sparsification(void* c, void* t, void* accumulation, float spars, int topk) {
  singa::Communicator* comm = static_cast<singa::Communicator*>(c);
  if (accumulation)
    comm->sparsification(T(t), T(accumulation), spars, topk != 0);
  else
    comm->sparsification(T(t), spars, topk != 0);
}
void rs_comm_wait(void* c) { static_cast<singa::Communicator*>(c)->wait(); }

}  // extern "C"
