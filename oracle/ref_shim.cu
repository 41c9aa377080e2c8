// extern "C" doors into the reference's own CUDA launchers (namespace
// singa::cuda, declared in apache/singa src/core/tensor/math_kernel.h), so
// that the test-suite can run the UNMODIFIED reference kernels next to the new
// ones on the same device buffers.  TEST INFRASTRUCTURE ONLY: this file is
// compiled together with the reference's math_kernel.cu (read from the
// reference tree, never copied) into oracle/_ref/libref_cuda.so by
// oracle/ref_build.py.  Only launchers whose behaviour is defined are exposed
// (removezeroidx is not: it counts over unspecified memory).
#include "math_kernel.h"

#define S static_cast<cudaStream_t>(stream)
using namespace singa::cuda;

extern "C" {
void ref_relu(size_t n, const float* in, float* out, void* stream) { relu(n, in, out, S); }
void ref_relubackward(size_t n, const float* in1, const float* in2, float* out, void* stream) {
  relubackward(n, in1, in2, out, S);
}
void ref_relu_half(size_t n, const void* in, void* out, void* stream) {
  relu(n, static_cast<const __half*>(in), static_cast<__half*>(out), S);
}
void ref_relubackward_half(size_t n, const void* in1, const void* in2, void* out, void* stream) {
  relubackward(n, static_cast<const __half*>(in1), static_cast<const __half*>(in2),
               static_cast<__half*>(out), S);
}
void ref_add(size_t n, const float* a, const float* b, float* out, void* stream) { add(n, a, b, out, S); }
void ref_sub(size_t n, const float* a, const float* b, float* out, void* stream) { sub(n, a, b, out, S); }
void ref_mult(size_t n, const float* a, const float* b, float* out, void* stream) { mult(n, a, b, out, S); }
void ref_div(size_t n, const float* a, const float* b, float* out, void* stream) { div(n, a, b, out, S); }
void ref_mult_scalar(size_t n, const float* a, float x, float* out, void* stream) { mult(n, a, x, out, S); }
void ref_add_scalar(size_t n, const float* a, float x, float* out, void* stream) { add(n, a, x, out, S); }
void ref_exp(size_t n, const float* a, float* out, void* stream) { singa::cuda::exp(n, a, out, S); }
void ref_log(size_t n, const float* a, float* out, void* stream) { singa::cuda::log(n, a, out, S); }
void ref_sqrt(size_t n, const float* a, float* out, void* stream) { singa::cuda::sqrt(n, a, out, S); }
void ref_tanh(size_t n, const float* a, float* out, void* stream) { singa::cuda::tanh(n, a, out, S); }
void ref_sigmoid(size_t n, const float* a, float* out, void* stream) { sigmoid(n, a, out, S); }
void ref_float2half(size_t n, const float* in, void* out, void* stream) {
  float2half(n, in, static_cast<__half*>(out), S);
}
void ref_half2float(size_t n, const void* in, float* out, void* stream) {
  half2float(n, static_cast<const __half*>(in), out, S);
}
void ref_sparsabs(size_t n, float thr, const float* in, float* out, void* stream) {
  sparsabs(n, thr, in, out, S);
}
void ref_sparsindex(size_t n, const float* in, int* out, void* stream) { sparsindex(n, in, out, S); }
void ref_generateindex(size_t n, int* out, void* stream) { generateindex(n, out, S); }
void ref_sortbykey(size_t n, float* key, int* value, void* stream) { sortbykey(n, key, value, S); }
void ref_cross_entropy(int int_target, size_t batch, size_t dim, const float* p, const int* t,
                       float* loss, void* stream) {
  ComputeCrossEntropy(int_target != 0, batch, dim, p, t, loss, S);
}
void ref_softmax_cross_entropy_bwd(int int_target, size_t batch, size_t dim, const float* p,
                                   const int* t, float* grad, void* stream) {
  SoftmaxCrossEntropyBwd(int_target != 0, batch, dim, p, t, grad, S);
}
void ref_row_max(size_t nrow, size_t ncol, const float* in, float* out, void* stream) {
  RowMax(nrow, ncol, in, out, S);
}
}
