// Row softmax, per-sample cross entropy and the softmax-cross-entropy gradient.
// The problems on this path are tiny (batch x classes = 32x1000 ... 256x10), so
// the point of these kernels is to be ONE launch each and to fold the 1/batch
// scaling into the gradient instead of a clone + edit + scale sequence.
#include <float.h>

#include "common.cuh"

namespace sgb {
namespace {

constexpr int kBlock = 128;

// One CTA per row: max, sum of exp(x - max), normalise.  expf and the division
// are the full-precision forms (the "accurate" softmax mode).
__global__ void __launch_bounds__(kBlock)
softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, size_t ncol) {
  __shared__ float sm[32];
  const float* xr = x + blockIdx.x * ncol;
  float* yr = y + blockIdx.x * ncol;
  float m = xr[0];
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) m = fmaxf(m, xr[c]);
  m = warp_max(m);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sm[w] = m;
  __syncthreads();
  m = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
  float s = 0.f;
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) s += expf(xr[c] - m);
  s = block_sum(s, sm);
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) yr[c] = expf(xr[c] - m) / s;
}

// loss[i] = -log(max(p[i, t[i]], FLT_MIN)) or the weighted form for array
// targets; one thread per sample like the reference (batch is small).
__global__ void ce_fwd_kernel(int int_target, size_t batch, size_t dim,
                              const float* __restrict__ p, const int* __restrict__ t,
                              float* __restrict__ loss) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= batch) return;
  if (int_target) {
    // a label outside [0, dim) reads nothing: the sample's loss is NaN
    const int ti = t[i];
    if (static_cast<unsigned>(ti) >= dim) {
      loss[i] = __int_as_float(0x7fc00000);
      return;
    }
    float pt = p[i * dim + ti];
    loss[i] = -logf(fmaxf(pt, FLT_MIN));
  } else {
    float sum = 0.f;
    for (size_t j = 0; j < dim; ++j) sum += t[i * dim + j];
    float l = 0.f;
    for (size_t j = 0; j < dim; ++j)
      l -= t[i * dim + j] / sum * logf(fmaxf(p[i * dim + j], FLT_MIN));
    loss[i] = l;
  }
}

// grad = (p - target) * scale, one CTA per sample row.  With SCALE == false the
// multiply is skipped, so the values equal the reference's in-place kernel bit
// for bit; with SCALE the extra multiply is the same fp32 product the
// reference forms in its separate "dx /= batch" pass.
template <bool SCALE>
__global__ void __launch_bounds__(kBlock)
ce_bwd_kernel(int int_target, size_t dim, const float* __restrict__ p,
              const int* __restrict__ t, float* __restrict__ grad, float scale) {
  __shared__ float sm[32];
  const size_t row = blockIdx.x;
  const float* pr = p + row * dim;
  float* gr = grad + row * dim;
  if (int_target) {
    const size_t hot = static_cast<size_t>(t[row]);
    for (size_t j = threadIdx.x; j < dim; j += kBlock) {
      float g = pr[j];
      if (j == hot) g = g - 1.0f;
      gr[j] = SCALE ? g * scale : g;
    }
  } else {
    const int* tr = t + row * dim;
    // the reference adds the integer weights serially in fp32; sums of small
    // integers are exact in any order
    float part = 0.f;
    for (size_t j = threadIdx.x; j < dim; j += kBlock) part += tr[j];
    const float sum = block_sum(part, sm);
    for (size_t j = threadIdx.x; j < dim; j += kBlock) {
      float g = pr[j] - tr[j] / sum;
      gr[j] = SCALE ? g * scale : g;
    }
  }
}

// The whole loss head for integer targets in one launch, one CTA per sample:
// row softmax, the sample's loss -log(max(p[t], FLT_MIN)) and the scaled
// gradient (p - onehot) * scale.  Every value is formed by the same fp32
// operations as in the three separate kernels above, so results are identical
// bit for bit.
__global__ void __launch_bounds__(kBlock)
softmax_ce_fused_kernel(const float* __restrict__ x, const int* __restrict__ t,
                        float* __restrict__ prob, float* __restrict__ loss,
                        float* __restrict__ grad, size_t ncol, float scale) {
  __shared__ float sm[32];
  const size_t row = blockIdx.x;
  const float* xr = x + row * ncol;
  float m = xr[0];
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) m = fmaxf(m, xr[c]);
  m = warp_max(m);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sm[w] = m;
  __syncthreads();
  m = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
  float s = 0.f;
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) s += expf(xr[c] - m);
  s = block_sum(s, sm);
  const size_t hot = static_cast<size_t>(t[row]);
  if (hot >= ncol && threadIdx.x == 0) loss[row] = __int_as_float(0x7fc00000);   // label out of range: NaN, not stale memory
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) {
    const float p = expf(xr[c] - m) / s;
    if (prob) prob[row * ncol + c] = p;
    float g = p;
    if (c == hot) {
      g = g - 1.0f;
      loss[row] = -logf(fmaxf(p, FLT_MIN));
    }
    grad[row * ncol + c] = g * scale;
  }
}

// ------------------------------------------------------------------- fp16
// Row softmax on fp16 data: fp32 arithmetic inside, one rounding on store.
__global__ void __launch_bounds__(kBlock)
softmax_rows_f16_kernel(const __half* __restrict__ x, __half* __restrict__ y, size_t ncol) {
  __shared__ float sm[32];
  const __half* xr = x + blockIdx.x * ncol;
  __half* yr = y + blockIdx.x * ncol;
  float m = __half2float(xr[0]);
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) m = fmaxf(m, __half2float(xr[c]));
  m = warp_max(m);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sm[w] = m;
  __syncthreads();
  m = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
  float s = 0.f;
  for (size_t c = threadIdx.x; c < ncol; c += kBlock) s += expf(__half2float(xr[c]) - m);
  s = block_sum(s, sm);
  for (size_t c = threadIdx.x; c < ncol; c += kBlock)
    yr[c] = __float2half_rn(expf(__half2float(xr[c]) - m) / s);
}

// fp16 cross entropy with the arithmetic of the fp16 kernel it replaces: all
// steps in half precision, probabilities floored at half(1e-7), integer
// weights converted with round-down, the per-sample sums formed serially.
__global__ void ce_fwd_f16_kernel(int int_target, size_t batch, size_t dim,
                                  const __half* __restrict__ p, const int* __restrict__ t,
                                  __half* __restrict__ loss) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= batch) return;
  const __half eps = __float2half_rn(0.0000001f);
  if (int_target) {
    const int ti = t[i];
    if (static_cast<unsigned>(ti) >= dim) {      // label out of range: NaN, no read
      loss[i] = __ushort_as_half(0x7e00);
      return;
    }
    const __half pt = p[i * dim + ti];
    loss[i] = __hneg(hlog(__hgt(pt, eps) ? pt : eps));
  } else {
    __half sum = __float2half_rn(0.f);
    for (size_t j = 0; j < dim; ++j) sum = __hadd(sum, __int2half_rd(t[i * dim + j]));
    __half l = __float2half_rn(0.f);
    for (size_t j = 0; j < dim; ++j) {
      const __half pj = p[i * dim + j];
      l = __hsub(l, __hmul(__hdiv(__int2half_rd(t[i * dim + j]), sum), hlog(__hgt(pj, eps) ? pj : eps)));
    }
    loss[i] = l;
  }
}

// grad = p - target in half precision; one CTA per sample row.  The integer
// weights of an array target are small, so their half sum is exact in any
// order as long as it stays below 2048.
__global__ void __launch_bounds__(kBlock)
ce_bwd_f16_kernel(int int_target, size_t dim, const __half* __restrict__ p,
                  const int* __restrict__ t, __half* __restrict__ grad) {
  __shared__ __half total;
  const size_t row = blockIdx.x;
  const __half* pr = p + row * dim;
  __half* gr = grad + row * dim;
  if (int_target) {
    const size_t hot = static_cast<size_t>(t[row]);
    for (size_t j = threadIdx.x; j < dim; j += kBlock)
      gr[j] = j == hot ? __hsub(pr[j], __int2half_rn(1)) : pr[j];
  } else {
    const int* tr = t + row * dim;
    if (threadIdx.x == 0) {
      __half sum = __float2half_rn(0.f);
      for (size_t j = 0; j < dim; ++j) sum = __hadd(sum, __int2half_rd(tr[j]));
      total = sum;
    }
    __syncthreads();
    for (size_t j = threadIdx.x; j < dim; j += kBlock)
      gr[j] = __hsub(pr[j], __hdiv(__int2half_rd(tr[j]), total));
  }
}

}  // namespace
}  // namespace sgb

using namespace sgb;

extern "C" {

int sgb_softmax_rows_f32(const float* x, float* y, size_t nrow, size_t ncol, void* stream) {
  if (nrow == 0 || ncol == 0) return SGB_OK;
  if (!x || !y) return SGB_ERR_NULL;
  if (nrow > 0x7fffffffu) return SGB_ERR_SIZE;
  softmax_rows_kernel<<<static_cast<unsigned>(nrow), kBlock, 0, as_stream(stream)>>>(x, y, ncol);
  return launch_status();
}

int sgb_cross_entropy_f32(int int_target, size_t batch, size_t dim, const float* p,
                          const int32_t* t, float* loss, void* stream) {
  if (batch == 0) return SGB_OK;
  if (!p || !t || !loss) return SGB_ERR_NULL;
  if (dim == 0) return SGB_ERR_SIZE;
  ce_fwd_kernel<<<static_cast<unsigned>(ceil_div(batch, 128)), 128, 0, as_stream(stream)>>>(
      int_target, batch, dim, p, t, loss);
  return launch_status();
}

int sgb_softmax_cross_entropy_bwd_f32(int int_target, size_t batch, size_t dim, const float* p,
                                      const int32_t* t, float* grad, void* stream) {
  if (batch == 0 || dim == 0) return SGB_OK;
  if (!p || !t || !grad) return SGB_ERR_NULL;
  if (batch > 0x7fffffffu) return SGB_ERR_SIZE;
  ce_bwd_kernel<false><<<static_cast<unsigned>(batch), kBlock, 0, as_stream(stream)>>>(
      int_target, dim, p, t, grad, 1.0f);
  return launch_status();
}

int sgb_softmax_cross_entropy_grad_f32(int int_target, size_t batch, size_t dim, const float* p,
                                       const int32_t* t, float scale, float* grad, void* stream) {
  if (batch == 0 || dim == 0) return SGB_OK;
  if (!p || !t || !grad) return SGB_ERR_NULL;
  if (batch > 0x7fffffffu) return SGB_ERR_SIZE;
  ce_bwd_kernel<true><<<static_cast<unsigned>(batch), kBlock, 0, as_stream(stream)>>>(
      int_target, dim, p, t, grad, scale);
  return launch_status();
}

int sgb_softmax_cross_entropy_fused_f32(const float* logits, const int32_t* t, size_t batch, size_t dim,
                                        float scale, float* prob, float* loss, float* grad,
                                        void* stream) {
  if (batch == 0 || dim == 0) return SGB_OK;
  if (!logits || !t || !loss || !grad) return SGB_ERR_NULL;
  if (batch > 0x7fffffffu) return SGB_ERR_SIZE;
  softmax_ce_fused_kernel<<<static_cast<unsigned>(batch), kBlock, 0, as_stream(stream)>>>(
      logits, t, prob, loss, grad, dim, scale);
  return launch_status();
}

int sgb_softmax_rows_f16(const void* x, void* y, size_t nrow, size_t ncol, void* stream) {
  if (nrow == 0 || ncol == 0) return SGB_OK;
  if (!x || !y) return SGB_ERR_NULL;
  if (nrow > 0x7fffffffu) return SGB_ERR_SIZE;
  softmax_rows_f16_kernel<<<static_cast<unsigned>(nrow), kBlock, 0, as_stream(stream)>>>(
      static_cast<const __half*>(x), static_cast<__half*>(y), ncol);
  return launch_status();
}

int sgb_cross_entropy_f16(int int_target, size_t batch, size_t dim, const void* p, const int32_t* t,
                          void* loss, void* stream) {
  if (batch == 0) return SGB_OK;
  if (!p || !t || !loss) return SGB_ERR_NULL;
  if (dim == 0) return SGB_ERR_SIZE;
  ce_fwd_f16_kernel<<<static_cast<unsigned>(ceil_div(batch, 128)), 128, 0, as_stream(stream)>>>(
      int_target, batch, dim, static_cast<const __half*>(p), t, static_cast<__half*>(loss));
  return launch_status();
}

int sgb_softmax_cross_entropy_bwd_f16(int int_target, size_t batch, size_t dim, const void* p,
                                      const int32_t* t, void* grad, void* stream) {
  if (batch == 0 || dim == 0) return SGB_OK;
  if (!p || !t || !grad) return SGB_ERR_NULL;
  if (batch > 0x7fffffffu) return SGB_ERR_SIZE;
  ce_bwd_f16_kernel<<<static_cast<unsigned>(batch), kBlock, 0, as_stream(stream)>>>(
      int_target, dim, static_cast<const __half*>(p), t, static_cast<__half*>(grad));
  return launch_status();
}

}  // extern "C"
