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

#include <cub/device/device_radix_sort.cuh>

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

// ---- the three helpers the reference builds on Thrust (math_kernel.cu:704-727).
// They are kept for source compatibility only: the replacement communicator
// selects and compacts inside sgb_sparse_*, and calls none of them.  Like the
// Thrust versions they take no workspace, so their scratch comes from the
// stream-ordered allocator (cudaMallocAsync on `s`).
namespace {
constexpr int kTile = 2048, kCompactBlock = 256;

}  // namespace

// The compaction kernels treat the elements as 32-bit words; IS_FLOAT decides
// whether the bit pattern of -0.0f counts as zero.
namespace {
template <bool IS_FLOAT>
__device__ __forceinline__ bool nonzero(unsigned bits) {
  return IS_FLOAT ? (bits << 1) != 0u : bits != 0u;
}

template <bool IS_FLOAT>
__global__ void __launch_bounds__(kCompactBlock)
tile_count_kernel(const unsigned* __restrict__ in, size_t n, unsigned* __restrict__ counts) {
  __shared__ unsigned warp_tot[kCompactBlock / 32];
  const size_t base = static_cast<size_t>(blockIdx.x) * kTile;
  unsigned c = 0;
  for (int k = threadIdx.x; k < kTile; k += kCompactBlock)
    if (base + k < n && nonzero<IS_FLOAT>(in[base + k])) ++c;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned t = 0;
    for (int w = 0; w < kCompactBlock / 32; ++w) t += warp_tot[w];
    counts[blockIdx.x] = t;
  }
}

// Exclusive scan of the tile counts in place, one CTA; counts[tiles] = total.
__global__ void __launch_bounds__(1024) tile_scan_kernel(unsigned* __restrict__ counts, unsigned tiles) {
  __shared__ unsigned carry, warp_tot[32];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (unsigned base = 0; base < tiles; base += 1024) {
    const unsigned i = base + threadIdx.x;
    const unsigned v = i < tiles ? counts[i] : 0u;
    unsigned incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if ((threadIdx.x & 31) >= o) incl += t;
    }
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = incl;
    __syncthreads();
    if (threadIdx.x < 32) {
      unsigned w = warp_tot[threadIdx.x], wi = w;
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, wi, o);
        if (threadIdx.x >= o) wi += t;
      }
      warp_tot[threadIdx.x] = wi - w;            // exclusive prefix of the warp totals
    }
    __syncthreads();
    const unsigned excl = carry + warp_tot[threadIdx.x >> 5] + incl - v;
    if (i < tiles) counts[i] = excl;
    __syncthreads();
    if (threadIdx.x == 1023) carry = excl + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[tiles] = carry;
}

// Writes the non-zero elements of each tile, in order, at the tile's offset.
template <bool IS_FLOAT>
__global__ void __launch_bounds__(kCompactBlock)
tile_write_kernel(const unsigned* __restrict__ in, size_t n, const unsigned* __restrict__ offsets,
                  unsigned* __restrict__ out) {
  __shared__ unsigned warp_base[kCompactBlock / 32], running;
  const size_t base = static_cast<size_t>(blockIdx.x) * kTile;
  if (threadIdx.x == 0) running = offsets[blockIdx.x];
  __syncthreads();
  for (int k0 = 0; k0 < kTile; k0 += kCompactBlock) {
    const size_t i = base + k0 + threadIdx.x;
    const unsigned v = i < n ? in[i] : 0u;
    const bool keep = i < n && nonzero<IS_FLOAT>(v);
    const unsigned ballot = __ballot_sync(0xffffffffu, keep);
    const unsigned lane = threadIdx.x & 31, rank = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_base[threadIdx.x >> 5] = __popc(ballot);
    __syncthreads();
    unsigned before = running;
    for (int w = 0; w < (threadIdx.x >> 5); ++w) before += warp_base[w];
    if (keep) out[before + rank] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned t = 0;
      for (int w = 0; w < kCompactBlock / 32; ++w) t += warp_base[w];
      running += t;
    }
    __syncthreads();
  }
}

__global__ void copy_prefix_kernel(const unsigned* __restrict__ src, const unsigned* __restrict__ total,
                                   unsigned* __restrict__ dst) {
  const unsigned t = *total;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < t;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

inline void must_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    std::fprintf(stderr, "singa::cuda::%s failed: %s\n", what, cudaGetErrorString(e));
    std::abort();
  }
}

// Stable in-place removal of zeros from n 32-bit elements; returns the number kept when asked.
template <bool IS_FLOAT>
void compact_nonzero(size_t n, unsigned* data, cudaStream_t s, int* kept_host, const char* who) {
  if (n == 0) {
    if (kept_host) *kept_host = 0;
    return;
  }
  const unsigned tiles = static_cast<unsigned>((n + kTile - 1) / kTile);
  unsigned *tmp = nullptr, *counts = nullptr;
  must_cuda(cudaMallocAsync(&tmp, n * sizeof(unsigned), s), who);
  must_cuda(cudaMallocAsync(&counts, (static_cast<size_t>(tiles) + 1) * sizeof(unsigned), s), who);
  tile_count_kernel<IS_FLOAT><<<tiles, kCompactBlock, 0, s>>>(data, n, counts);
  tile_scan_kernel<<<1, 1024, 0, s>>>(counts, tiles);
  tile_write_kernel<IS_FLOAT><<<tiles, kCompactBlock, 0, s>>>(data, n, counts, tmp);
  copy_prefix_kernel<<<148 * 8, 256, 0, s>>>(tmp, counts + tiles, data);
  must_cuda(cudaGetLastError(), who);
  if (kept_host) {
    unsigned kept = 0;
    must_cuda(cudaMemcpyAsync(&kept, counts + tiles, sizeof(unsigned), cudaMemcpyDeviceToHost, s), who);
    must_cuda(cudaStreamSynchronize(s), who);
    *kept_host = static_cast<int>(kept);
  }
  must_cuda(cudaFreeAsync(tmp, s), who);
  must_cuda(cudaFreeAsync(counts, s), who);
}
}  // namespace

/// in[0 .. kept) = the non-zero values of in, in their original order.
void removezeroval(const size_t n, float* in, cudaStream_t s) {
  compact_nonzero<true>(n, reinterpret_cast<unsigned*>(in), s, nullptr, "removezeroval");
}
/// The same for indices; *address receives the number of non-zero entries -
/// what the reference's caller needs.  (The reference counts zeros over the
/// whole array after thrust::remove, whose tail is unspecified.)
void removezeroidx(const size_t n, int* in, cudaStream_t s, int* address) {
  compact_nonzero<false>(n, reinterpret_cast<unsigned*>(in), s, address, "removezeroidx");
}

namespace {
// The reference's comparator orders by max((int)v, -(int)v), descending.
__global__ void sort_keys_kernel(const float* __restrict__ key, size_t n, unsigned* __restrict__ k2,
                                 unsigned* __restrict__ pos) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(key[i]);
    k2[i] = static_cast<unsigned>(t > -t ? t : -t);
    pos[i] = static_cast<unsigned>(i);
  }
}
__global__ void permute_kernel(const unsigned* __restrict__ pos, size_t n, const float* __restrict__ key,
                               const int* __restrict__ value, float* __restrict__ key_out,
                               int* __restrict__ value_out) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    key_out[i] = key[pos[i]];
    value_out[i] = value[pos[i]];
  }
}
}  // namespace

/// Sorts (key, value) pairs by the reference's comparator (absgreater on the
/// integer-truncated keys), stably: equal keys keep their original order.
void sortbykey(const size_t n, float* key, int* value, cudaStream_t s) {
  if (n < 2) return;
  if (n > 0x7fffffffu) must(SGB_ERR_SIZE, "sortbykey");
  unsigned *k2 = nullptr, *k2_out = nullptr, *pos = nullptr, *pos_out = nullptr;
  float* key_out = nullptr;
  int* value_out = nullptr;
  void* cub_tmp = nullptr;
  size_t cub_bytes = 0;
  const int num = static_cast<int>(n);
  must_cuda(cub::DeviceRadixSort::SortPairsDescending(nullptr, cub_bytes, k2, k2_out, pos, pos_out, num, 0, 32, s),
            "sortbykey");
  must_cuda(cudaMallocAsync(&k2, n * 4, s), "sortbykey");
  must_cuda(cudaMallocAsync(&k2_out, n * 4, s), "sortbykey");
  must_cuda(cudaMallocAsync(&pos, n * 4, s), "sortbykey");
  must_cuda(cudaMallocAsync(&pos_out, n * 4, s), "sortbykey");
  must_cuda(cudaMallocAsync(&cub_tmp, cub_bytes ? cub_bytes : 4, s), "sortbykey");
  sort_keys_kernel<<<148 * 8, 256, 0, s>>>(key, n, k2, pos);
  must_cuda(cub::DeviceRadixSort::SortPairsDescending(cub_tmp, cub_bytes, k2, k2_out, pos, pos_out, num, 0, 32, s),
            "sortbykey");
  // k2 / pos are free again: reuse them for the permuted pairs
  key_out = reinterpret_cast<float*>(k2);
  value_out = reinterpret_cast<int*>(pos);
  permute_kernel<<<148 * 8, 256, 0, s>>>(pos_out, n, key, value, key_out, value_out);
  must_cuda(cudaMemcpyAsync(key, key_out, n * 4, cudaMemcpyDeviceToDevice, s), "sortbykey");
  must_cuda(cudaMemcpyAsync(value, value_out, n * 4, cudaMemcpyDeviceToDevice, s), "sortbykey");
  must_cuda(cudaGetLastError(), "sortbykey");
  for (void* b : {static_cast<void*>(k2), static_cast<void*>(k2_out), static_cast<void*>(pos),
                  static_cast<void*>(pos_out), cub_tmp})
    must_cuda(cudaFreeAsync(b, s), "sortbykey");
}

}  // namespace cuda
}  // namespace singa
