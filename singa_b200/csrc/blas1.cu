// BLAS-1 style reductions (dot, sum |x|, 2-norm, arg max / min of |x|), the
// diagonal scaling DGMM and the fp16 axpy.  They stand in for the cuBLAS calls
// behind Dot / Asum / Nrm2 / Amax / Amin / DGMM / Axpy<half> of the CUDA
// tensor backend, with two differences that matter on the training path: the
// result always lands in DEVICE memory (no host round trip, so the call can
// sit inside a captured graph) and the summation order is fixed (partials per
// CTA, then one CTA in index order), so results repeat run to run.
#include <float.h>

#include "common.cuh"

namespace sgb {
namespace {

constexpr int kBlock = 256;
constexpr int kMaxParts = 1024;

enum Kind { kDot = 0, kAsum = 1, kSumSq = 2 };

inline int parts_for(size_t n) {
  size_t p = ceil_div(n, static_cast<size_t>(kBlock) * 16);
  size_t cap = static_cast<size_t>(sm_count()) * 4;
  if (cap > kMaxParts) cap = kMaxParts;
  if (p > cap) p = cap;
  return static_cast<int>(p < 1 ? 1 : p);
}

template <int KIND>
__device__ __forceinline__ float term(float a, float b) {
  if (KIND == kDot) return a * b;
  if (KIND == kAsum) return fabsf(a);
  return a * a;
}

// Partial sums, one per CTA.  VEC: both operands 16-byte aligned; the tail
// (n % 4 elements) is added by CTA 0.
template <int KIND, bool VEC>
__global__ void __launch_bounds__(kBlock)
sum_partial_kernel(const float* __restrict__ x, const float* __restrict__ y,
                   float* __restrict__ partial, size_t n) {
  __shared__ float sm[32];
  float acc = 0.f;
  const size_t tid = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x;
  const size_t step = static_cast<size_t>(gridDim.x) * kBlock;
  if (VEC) {
    const size_t n4 = n >> 2;
    for (size_t i = tid; i < n4; i += step) {
      Vec4f a, b;
      a.u = ld128(x + 4 * i);
      if (KIND == kDot) b.u = ld128(y + 4 * i);
      else b = a;
      acc += (term<KIND>(a.f[0], b.f[0]) + term<KIND>(a.f[1], b.f[1])) +
             (term<KIND>(a.f[2], b.f[2]) + term<KIND>(a.f[3], b.f[3]));
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
      const size_t i = (n4 << 2) + threadIdx.x;
      acc += term<KIND>(x[i], KIND == kDot ? y[i] : 0.f);
    }
  } else {
    for (size_t i = tid; i < n; i += step) acc += term<KIND>(x[i], KIND == kDot ? y[i] : 0.f);
  }
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

template <bool ROOT>
__global__ void __launch_bounds__(kBlock)
sum_finish_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts) {
  __shared__ float sm[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < parts; i += kBlock) acc += partial[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) out[0] = ROOT ? sqrtf(acc) : acc;
}

// (|x|, index) candidates.  MAX: largest |x|; otherwise smallest.  Ties go to
// the lowest index (the first occurrence, as cublasIsamax / Isamin report).
struct Cand {
  float v;
  unsigned idx;
};
template <bool MAX>
__device__ __forceinline__ bool better(float v, unsigned i, float bv, unsigned bi) {
  return MAX ? (v > bv || (v == bv && i < bi)) : (v < bv || (v == bv && i < bi));
}
template <bool MAX>
__device__ __forceinline__ Cand block_best(Cand c, Cand* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, c.v, o);
    const unsigned oi = __shfl_xor_sync(0xffffffffu, c.idx, o);
    if (better<MAX>(ov, oi, c.v, c.idx)) {
      c.v = ov;
      c.idx = oi;
    }
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sm[wid] = c;
  __syncthreads();
  if (wid == 0) {
    Cand d = lane < kBlock / 32 ? sm[lane] : Cand{MAX ? -1.0f : INFINITY, 0xffffffffu};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, d.v, o);
      const unsigned oi = __shfl_xor_sync(0xffffffffu, d.idx, o);
      if (better<MAX>(ov, oi, d.v, d.idx)) {
        d.v = ov;
        d.idx = oi;
      }
    }
    c = d;
  }
  return c;   // valid in warp 0
}

template <bool MAX>
__global__ void __launch_bounds__(kBlock)
arg_partial_kernel(const float* __restrict__ x, Cand* __restrict__ partial, size_t n) {
  __shared__ Cand sm[kBlock / 32];
  Cand c{MAX ? -1.0f : INFINITY, 0xffffffffu};
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    const float v = fabsf(x[i]);
    if (better<MAX>(v, static_cast<unsigned>(i), c.v, c.idx)) {
      c.v = v;
      c.idx = static_cast<unsigned>(i);
    }
  }
  c = block_best<MAX>(c, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = c;
}

template <bool MAX>
__global__ void __launch_bounds__(kBlock)
arg_finish_kernel(const Cand* __restrict__ partial, int32_t* __restrict__ out, int parts) {
  __shared__ Cand sm[kBlock / 32];
  Cand c{MAX ? -1.0f : INFINITY, 0xffffffffu};
  for (int i = threadIdx.x; i < parts; i += kBlock) {
    const Cand p = partial[i];
    if (better<MAX>(p.v, p.idx, c.v, c.idx)) c = p;
  }
  c = block_best<MAX>(c, sm);
  if (threadIdx.x == 0) out[0] = static_cast<int32_t>(c.idx);
}

template <int KIND, bool ROOT>
int reduce_sum(const float* x, const float* y, float* out, size_t n, void* ws, size_t ws_bytes,
               void* stream) {
  if (!out) return SGB_ERR_NULL;
  if (n == 0) return sgb_set_f32(0.f, out, 1, stream);
  if (!x || (KIND == kDot && !y)) return SGB_ERR_NULL;
  const int parts = parts_for(n);
  if (!ws || ws_bytes < parts * sizeof(Cand)) return SGB_ERR_WORKSPACE;
  cudaStream_t s = as_stream(stream);
  float* partial = static_cast<float*>(ws);
  if (aligned16(x) && (KIND != kDot || aligned16(y)))
    sum_partial_kernel<KIND, true><<<parts, kBlock, 0, s>>>(x, y, partial, n);
  else
    sum_partial_kernel<KIND, false><<<parts, kBlock, 0, s>>>(x, y, partial, n);
  sum_finish_kernel<ROOT><<<1, kBlock, 0, s>>>(partial, out, parts);
  return launch_status();
}

template <bool MAX>
int reduce_arg(const float* x, int32_t* out, size_t n, void* ws, size_t ws_bytes, void* stream) {
  if (!out || !x) return SGB_ERR_NULL;
  if (n == 0 || n > 0x7fffffffu) return SGB_ERR_SIZE;
  const int parts = parts_for(n);
  if (!ws || ws_bytes < parts * sizeof(Cand)) return SGB_ERR_WORKSPACE;
  cudaStream_t s = as_stream(stream);
  Cand* partial = static_cast<Cand*>(ws);
  arg_partial_kernel<MAX><<<parts, kBlock, 0, s>>>(x, partial, n);
  arg_finish_kernel<MAX><<<1, kBlock, 0, s>>>(partial, out, parts);
  return launch_status();
}

// out[r][c] = M[r][c] * (RIGHT ? v[c] : v[r]), row-major.
template <bool RIGHT>
__global__ void __launch_bounds__(kBlock)
dgmm_kernel(const float* __restrict__ M, const float* __restrict__ v, float* __restrict__ out,
            size_t nrow, size_t ncol) {
  const size_t n = nrow * ncol;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * kBlock) {
    const size_t r = i / ncol;
    out[i] = M[i] * v[RIGHT ? i - r * ncol : r];
  }
}

// y = half(alpha * float(x) + float(y)): one fp32 fused multiply-add and one
// rounding to fp16 per element (the AxpyEx contract with fp32 execution type).
template <bool DEV>
__global__ void __launch_bounds__(kBlock)
axpy_f16_kernel(float alpha, const float* __restrict__ alpha_dev, const __half* __restrict__ x,
                __half* __restrict__ y, size_t n) {
  const float a = DEV ? alpha_dev[0] : alpha;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * kBlock)
    y[i] = __float2half_rn(fmaf(a, __half2float(x[i]), __half2float(y[i])));
}

}  // namespace
}  // namespace sgb

using namespace sgb;

extern "C" {

size_t sgb_blas1_workspace_bytes(size_t n) {
  return n ? static_cast<size_t>(parts_for(n)) * sizeof(Cand) : 0;
}

int sgb_dot_f32(const float* x, const float* y, float* out, size_t n, void* ws, size_t ws_bytes,
                void* stream) {
  return reduce_sum<kDot, false>(x, y, out, n, ws, ws_bytes, stream);
}
int sgb_asum_f32(const float* x, float* out, size_t n, void* ws, size_t ws_bytes, void* stream) {
  return reduce_sum<kAsum, false>(x, nullptr, out, n, ws, ws_bytes, stream);
}
int sgb_nrm2_f32(const float* x, float* out, size_t n, void* ws, size_t ws_bytes, void* stream) {
  return reduce_sum<kSumSq, true>(x, nullptr, out, n, ws, ws_bytes, stream);
}
int sgb_amax_f32(const float* x, int32_t* index_out, size_t n, void* ws, size_t ws_bytes,
                 void* stream) {
  return reduce_arg<true>(x, index_out, n, ws, ws_bytes, stream);
}
int sgb_amin_f32(const float* x, int32_t* index_out, size_t n, void* ws, size_t ws_bytes,
                 void* stream) {
  return reduce_arg<false>(x, index_out, n, ws, ws_bytes, stream);
}

int sgb_dgmm_f32(int side_right, const float* M, const float* v, float* out, size_t nrow,
                 size_t ncol, void* stream) {
  if (nrow == 0 || ncol == 0) return SGB_OK;
  if (!M || !v || !out) return SGB_ERR_NULL;
  const unsigned grid = capped_grid(nrow * ncol, kBlock, 8);
  if (side_right)
    dgmm_kernel<true><<<grid, kBlock, 0, as_stream(stream)>>>(M, v, out, nrow, ncol);
  else
    dgmm_kernel<false><<<grid, kBlock, 0, as_stream(stream)>>>(M, v, out, nrow, ncol);
  return launch_status();
}

int sgb_axpy_f16(float alpha, const void* x, void* y, size_t n, void* stream) {
  if (n == 0) return SGB_OK;
  if (!x || !y) return SGB_ERR_NULL;
  axpy_f16_kernel<false><<<capped_grid(n, kBlock, 8), kBlock, 0, as_stream(stream)>>>(
      alpha, nullptr, static_cast<const __half*>(x), static_cast<__half*>(y), n);
  return launch_status();
}
int sgb_axpy_dev_alpha_f16(const float* alpha_dev, const void* x, void* y, size_t n, void* stream) {
  if (n == 0) return SGB_OK;
  if (!alpha_dev || !x || !y) return SGB_ERR_NULL;
  axpy_f16_kernel<true><<<capped_grid(n, kBlock, 8), kBlock, 0, as_stream(stream)>>>(
      0.f, alpha_dev, static_cast<const __half*>(x), static_cast<__half*>(y), n);
  return launch_status();
}

}  // extern "C"
