// Reductions of the backward path: bias gradients (column sums of a row-major
// matrix), row sums, per-channel sums of an NCHW tensor (convolution bias
// gradient), the scalar sum behind SumAll and the per-row maximum.
//
// All sums are formed in a fixed order (per-thread strided accumulation, warp
// shuffles, then a fixed-order combine of per-CTA partials), so results are
// identical from run to run; none uses atomics.
#include "common.cuh"

namespace sgb {
namespace {

constexpr int kBlock = 256;

// ---------------------------------------------------------------- column sums
// v[c] = sum_r M[r][c].  A CTA owns 32 adjacent columns (one per lane) and a
// slice of the rows (blockIdx.y); its 8 warps stride over the rows, so every
// warp-load is one coalesced 128-byte line.  With gridDim.y > 1 the CTA writes
// a partial row to `partial` and the second kernel adds the slices in order.
__global__ void __launch_bounds__(kBlock)
colsum_kernel(const float* __restrict__ M, float* __restrict__ out, size_t nrow,
              size_t ncol, size_t rows_per_slice) {
  __shared__ float sm[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const size_t c = blockIdx.x * 32ull + lane;
  const size_t r0 = blockIdx.y * rows_per_slice;
  const size_t r1 = r0 + rows_per_slice < nrow ? r0 + rows_per_slice : nrow;
  float acc = 0.f;
  if (c < ncol)
    for (size_t r = r0 + w; r < r1; r += 8) acc += M[r * ncol + c];
  sm[w][lane] = acc;
  __syncthreads();
  if (w == 0 && c < ncol) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += sm[k][lane];
    out[blockIdx.y * ncol + c] = s;
  }
}

__global__ void __launch_bounds__(kBlock)
colsum_finish_kernel(const float* __restrict__ partial, float* __restrict__ v,
                     size_t ncol, int slices) {
  const size_t c = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x;
  if (c >= ncol) return;
  float s = 0.f;
  for (int k = 0; k < slices; ++k) s += partial[k * ncol + c];
  v[c] = s;
}

int colsum_slices(size_t nrow, size_t ncol) {
  const size_t col_blocks = ceil_div(ncol, 32);
  const size_t target = static_cast<size_t>(sm_count()) * 4;
  size_t s = col_blocks >= target ? 1 : ceil_div(target, col_blocks);
  const size_t max_by_rows = ceil_div(nrow, 64);  // at least 64 rows per slice
  if (s > max_by_rows) s = max_by_rows;
  if (s > 256) s = 256;
  return static_cast<int>(s < 1 ? 1 : s);
}

// ------------------------------------------------------------------- row sums
// v[r] = sum_c M[r][c]; one warp per row, lanes stride over the columns.
__global__ void __launch_bounds__(kBlock)
rowsum_kernel(const float* __restrict__ M, float* __restrict__ v, size_t nrow, size_t ncol) {
  const int lane = threadIdx.x & 31;
  const size_t r = (blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x) >> 5;
  if (r >= nrow) return;
  const float* row = M + r * ncol;
  float acc = 0.f;
  for (size_t c = lane; c < ncol; c += 32) acc += row[c];
  acc = warp_sum(acc);
  if (lane == 0) v[r] = acc;
}

__global__ void __launch_bounds__(kBlock)
rowmax_kernel(const float* __restrict__ M, float* __restrict__ v, size_t nrow, size_t ncol) {
  const int lane = threadIdx.x & 31;
  const size_t r = (blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x) >> 5;
  if (r >= nrow) return;
  const float* row = M + r * ncol;
  float m = row[0];  // seeded with the first element, as the CUDA reference does
  for (size_t c = lane; c < ncol; c += 32) m = fmaxf(m, row[c]);
  m = warp_max(m);
  if (lane == 0) v[r] = m;
}

// ---------------------------------------------------- per-channel NCHW reduce
// db[c] = sum over n and the HW plane of dy[n][c][:].  grid = (slices, C); a
// CTA walks the flattened (n, i) index space of its channel slice.
__global__ void __launch_bounds__(kBlock)
chansum_kernel(const float* __restrict__ dy, float* __restrict__ out, int N, int C,
               int HW, int per_slice, int vec) {
  __shared__ float sm[32];
  const int c = blockIdx.y, slice = blockIdx.x;
  float acc = 0.f;
  if (vec) {
    const int hw4 = HW >> 2, total = N * hw4;
    int i0 = slice * per_slice, i1 = min(i0 + per_slice, total);
    for (int i = i0 + threadIdx.x; i < i1; i += kBlock) {
      const int n = i / hw4, q = i - n * hw4;
      const float4 v = *reinterpret_cast<const float4*>(
          dy + (static_cast<size_t>(n) * C + c) * HW + 4 * q);
      acc += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    const int total = N * HW;
    int i0 = slice * per_slice, i1 = min(i0 + per_slice, total);
    for (int i = i0 + threadIdx.x; i < i1; i += kBlock) {
      const int n = i / HW, q = i - n * HW;
      acc += dy[(static_cast<size_t>(n) * C + c) * HW + q];
    }
  }
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) out[static_cast<size_t>(c) * gridDim.x + slice] = acc;
}

__global__ void chansum_finish_kernel(const float* __restrict__ partial,
                                      float* __restrict__ db, int C, int slices) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int k = 0; k < slices; ++k) s += partial[static_cast<size_t>(c) * slices + k];
  db[c] = s;
}

int chan_slices(int N, int C, int HW) {
  const long long per_channel = static_cast<long long>(N) * HW;
  long long s = ceil_div(static_cast<size_t>(sm_count()) * 8, static_cast<size_t>(C));
  const long long max_s = (per_channel + 4095) / 4096;  // >= 4096 elements per slice
  if (s > max_s) s = max_s;
  if (s > 64) s = 64;
  return static_cast<int>(s < 1 ? 1 : s);
}

// ------------------------------------------------------------------ total sum
__global__ void __launch_bounds__(kBlock)
sumall_partial_kernel(const float* __restrict__ x, float* __restrict__ partial, size_t n) {
  __shared__ float sm[32];
  float acc = 0.f;
  for (size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * kBlock)
    acc += x[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(kBlock)
sumall_finish_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts) {
  __shared__ float sm[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < parts; i += kBlock) acc += partial[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) out[0] = acc;
}
int sumall_parts(size_t n) {
  size_t p = ceil_div(n, static_cast<size_t>(kBlock) * 16);
  size_t cap = static_cast<size_t>(sm_count()) * 8;
  if (p > cap) p = cap;
  return static_cast<int>(p < 1 ? 1 : p);
}

}  // namespace
}  // namespace sgb

using namespace sgb;

extern "C" {

size_t sgb_sum_rows_workspace_bytes(size_t nrow, size_t ncol) {
  if (nrow == 0 || ncol == 0) return 0;
  int s = colsum_slices(nrow, ncol);
  return s > 1 ? static_cast<size_t>(s) * ncol * sizeof(float) : 0;
}

int sgb_sum_rows_f32(const float* M, float* v, size_t nrow, size_t ncol, void* ws,
                     size_t ws_bytes, void* stream) {
  if (ncol == 0) return SGB_OK;
  if (!v) return SGB_ERR_NULL;
  cudaStream_t s = as_stream(stream);
  if (nrow == 0) return sgb_set_f32(0.f, v, ncol, stream);
  if (!M) return SGB_ERR_NULL;
  const int slices = colsum_slices(nrow, ncol);
  const dim3 grid(static_cast<unsigned>(ceil_div(ncol, 32)), slices);
  if (grid.x > 0x7fffffffu) return SGB_ERR_SIZE;
  if (slices == 1) {
    colsum_kernel<<<grid, kBlock, 0, s>>>(M, v, nrow, ncol, nrow);
  } else {
    if (!ws || ws_bytes < static_cast<size_t>(slices) * ncol * sizeof(float))
      return SGB_ERR_WORKSPACE;
    float* partial = static_cast<float*>(ws);
    colsum_kernel<<<grid, kBlock, 0, s>>>(M, partial, nrow, ncol, ceil_div(nrow, slices));
    colsum_finish_kernel<<<static_cast<unsigned>(ceil_div(ncol, kBlock)), kBlock, 0, s>>>(
        partial, v, ncol, slices);
  }
  return launch_status();
}

int sgb_sum_columns_f32(const float* M, float* v, size_t nrow, size_t ncol, void* stream) {
  if (nrow == 0) return SGB_OK;
  if (!v) return SGB_ERR_NULL;
  if (ncol == 0) return sgb_set_f32(0.f, v, nrow, stream);
  if (!M) return SGB_ERR_NULL;
  rowsum_kernel<<<static_cast<unsigned>(ceil_div(nrow * 32, kBlock)), kBlock, 0, as_stream(stream)>>>(
      M, v, nrow, ncol);
  return launch_status();
}

int sgb_row_max_f32(const float* M, float* v, size_t nrow, size_t ncol, void* stream) {
  if (nrow == 0) return SGB_OK;
  if (!M || !v) return SGB_ERR_NULL;
  if (ncol == 0) return SGB_ERR_SIZE;
  rowmax_kernel<<<static_cast<unsigned>(ceil_div(nrow * 32, kBlock)), kBlock, 0, as_stream(stream)>>>(
      M, v, nrow, ncol);
  return launch_status();
}

size_t sgb_conv_bias_backward_workspace_bytes(int N, int C, int HW) {
  if (N <= 0 || C <= 0 || HW <= 0) return 0;
  return static_cast<size_t>(chan_slices(N, C, HW)) * C * sizeof(float);
}

int sgb_conv_bias_backward_f32(const float* dy, float* db, int N, int C, int HW, void* ws,
                               size_t ws_bytes, void* stream) {
  if (C <= 0) return C == 0 ? SGB_OK : SGB_ERR_SIZE;
  if (N < 0 || HW < 0) return SGB_ERR_SIZE;
  if (!db) return SGB_ERR_NULL;
  if (N == 0 || HW == 0) return sgb_set_f32(0.f, db, C, stream);
  if (!dy) return SGB_ERR_NULL;
  if (static_cast<long long>(N) * HW > 0x7fffffffLL || C > 65535) return SGB_ERR_SIZE;
  const int slices = chan_slices(N, C, HW);
  if (!ws || ws_bytes < static_cast<size_t>(slices) * C * sizeof(float)) return SGB_ERR_WORKSPACE;
  const int vec = (HW % 4 == 0) && aligned16(dy);
  const int total = vec ? N * (HW / 4) : N * HW;
  const int per_slice = static_cast<int>(ceil_div(total, slices));
  cudaStream_t s = as_stream(stream);
  float* partial = static_cast<float*>(ws);
  chansum_kernel<<<dim3(slices, C), kBlock, 0, s>>>(dy, partial, N, C, HW, per_slice, vec);
  chansum_finish_kernel<<<static_cast<unsigned>(ceil_div(C, 128)), 128, 0, s>>>(partial, db, C, slices);
  return launch_status();
}

size_t sgb_sum_all_workspace_bytes(size_t n) {
  return n ? static_cast<size_t>(sumall_parts(n)) * sizeof(float) : 0;
}

int sgb_sum_all_f32(const float* x, float* out, size_t n, void* ws, size_t ws_bytes, void* stream) {
  if (!out) return SGB_ERR_NULL;
  if (n == 0) return sgb_set_f32(0.f, out, 1, stream);
  if (!x) return SGB_ERR_NULL;
  const int parts = sumall_parts(n);
  if (!ws || ws_bytes < parts * sizeof(float)) return SGB_ERR_WORKSPACE;
  cudaStream_t s = as_stream(stream);
  float* partial = static_cast<float*>(ws);
  if (parts == 1) {
    // one CTA covers everything: its block sum IS the result (adding the zeros
    // of a second pass would not change a bit), so write it straight to `out`
    sumall_partial_kernel<<<1, kBlock, 0, s>>>(x, out, n);
    return launch_status();
  }
  sumall_partial_kernel<<<parts, kBlock, 0, s>>>(x, partial, n);
  sumall_finish_kernel<<<1, kBlock, 0, s>>>(partial, out, parts);
  return launch_status();
}

}  // extern "C"
