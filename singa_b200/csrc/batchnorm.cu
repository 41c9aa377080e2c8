// Batch-normalisation backward (training mode) with saved mean and saved
// inverse standard deviation:
//   dbias[c]  = sum dy
//   dscale[c] = sum dy * (x - mean[c]) * invstd[c]
//   dx        = scale[c] * invstd[c] *
//               (dy - dbias[c]/M - (x - mean[c]) * invstd[c] * dscale[c] / M)
// M = N*H*W (spatial mode, NCHW) or N (per-activation mode, N x D).
//
// Two-pass scheme, 20 bytes of HBM traffic per element when the tensor does
// not fit L2:
//   pass 1  grid (slices, C): a CTA walks its slice of the channel's flattened
//           (n, hw) space with 128-bit loads and leaves two partial sums in the
//           workspace (no atomics, fixed order -> run-to-run identical);
//   pass 2  grid (tiles, C): every CTA first adds the channel's <= 64 partials
//           in one warp (the same order in every CTA), then streams
//           dx for its 1024-element tile.  CTAs with blockIdx.x == 0 also store
//           dscale/dbias.
// The optional ReLU mask fuses "dy = relu_in > 0 ? dy : 0" (the backward of
// the ReLU that follows the BN layer) into both passes, which removes one
// full write + read of the intermediate gradient.
#include "common.cuh"

namespace sgb {
namespace {

constexpr int kBlock = 256;
constexpr int kMaxSlices = 64;

struct BnShape {
  int N, C, HW;
};

__host__ __device__ inline int bn_slices_for(long long per_channel, int C, int sms) {
  long long s = (static_cast<long long>(sms) * 16 + C - 1) / C;
  const long long max_s = (per_channel + 2047) / 2048;  // >= 2048 elements per slice
  if (s > max_s) s = max_s;
  if (s > kMaxSlices) s = kMaxSlices;
  return static_cast<int>(s < 1 ? 1 : s);
}

template <bool VEC, bool MASK>
__global__ void __launch_bounds__(kBlock)
bn_bwd_reduce_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                     const float* __restrict__ relu_in, const float* __restrict__ mean,
                     float2* __restrict__ partial, BnShape sh, int per_slice) {
  __shared__ float sm[32];
  const int c = blockIdx.y, slice = blockIdx.x;
  const float mu = mean[c];
  float s_dy = 0.f, s_dyx = 0.f;
  if (VEC) {
    const int hw4 = sh.HW >> 2, total = sh.N * hw4;
    const int i0 = slice * per_slice, i1 = min(i0 + per_slice, total);
    for (int i = i0 + threadIdx.x; i < i1; i += kBlock) {
      const int n = i / hw4, q = i - n * hw4;
      const size_t off = (static_cast<size_t>(n) * sh.C + c) * sh.HW + 4 * q;
      Vec4f vx, vg, vm;
      vx.u = ld128(x + off);
      vg.u = ld128(dy + off);
      if (MASK) vm.u = ld128(relu_in + off);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float g = vg.f[k];
        if (MASK) g = vm.f[k] > 0 ? g : 0.0f;
        s_dy += g;
        s_dyx += g * (vx.f[k] - mu);
      }
    }
  } else {
    const int total = sh.N * sh.HW;
    const int i0 = slice * per_slice, i1 = min(i0 + per_slice, total);
    for (int i = i0 + threadIdx.x; i < i1; i += kBlock) {
      const int n = i / sh.HW, q = i - n * sh.HW;
      const size_t off = (static_cast<size_t>(n) * sh.C + c) * sh.HW + q;
      float g = dy[off];
      if (MASK) g = relu_in[off] > 0 ? g : 0.0f;
      s_dy += g;
      s_dyx += g * (x[off] - mu);
    }
  }
  s_dy = block_sum(s_dy, sm);
  s_dyx = block_sum(s_dyx, sm);
  if (threadIdx.x == 0)
    partial[static_cast<size_t>(c) * gridDim.x + slice] = make_float2(s_dy, s_dyx);
}

template <bool VEC, bool MASK>
__global__ void __launch_bounds__(kBlock)
bn_bwd_apply_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                    const float* __restrict__ relu_in, const float* __restrict__ scale,
                    const float* __restrict__ mean, const float* __restrict__ invstd,
                    const float2* __restrict__ partial, int slices, float* __restrict__ dx,
                    float* __restrict__ dscale, float* __restrict__ dbias, BnShape sh) {
  __shared__ float coef[4];
  const int c = blockIdx.y;
  if (threadIdx.x < 32) {
    // add the channel's partials: lanes take slices lane, lane+32; fixed order
    float a = 0.f, b = 0.f;
    for (int k = threadIdx.x; k < slices; k += 32) {
      const float2 p = partial[static_cast<size_t>(c) * slices + k];
      a += p.x;
      b += p.y;
    }
    a = warp_sum(a);
    b = warp_sum(b);
    if (threadIdx.x == 0) {
      const float r = invstd[c];
      const float inv_m = 1.0f / (static_cast<float>(sh.N) * static_cast<float>(sh.HW));
      const float ds = b * r;
      coef[0] = scale[c] * r;       // k
      coef[1] = a * inv_m;          // mean of dy
      coef[2] = ds * r * inv_m;     // slope on (x - mean)
      coef[3] = mean[c];
      if (blockIdx.x == 0) {
        dscale[c] = ds;
        dbias[c] = a;
      }
    }
  }
  __syncthreads();
  const float k = coef[0], a = coef[1], b = coef[2], mu = coef[3];
  if (VEC) {
    const int hw4 = sh.HW >> 2, total = sh.N * hw4;
    const int i = blockIdx.x * kBlock + threadIdx.x;
    if (i < total) {
      const int n = i / hw4, q = i - n * hw4;
      const size_t off = (static_cast<size_t>(n) * sh.C + c) * sh.HW + 4 * q;
      Vec4f vx, vg, vm, o;
      vx.u = ld128(x + off);
      vg.u = ld128(dy + off);
      if (MASK) vm.u = ld128(relu_in + off);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float g = vg.f[j];
        if (MASK) g = vm.f[j] > 0 ? g : 0.0f;
        o.f[j] = k * (g - a - (vx.f[j] - mu) * b);
      }
      st128(dx + off, o.u);
    }
  } else {
    const int total = sh.N * sh.HW;
    const int i = blockIdx.x * kBlock + threadIdx.x;
    if (i < total) {
      const int n = i / sh.HW, q = i - n * sh.HW;
      const size_t off = (static_cast<size_t>(n) * sh.C + c) * sh.HW + q;
      float g = dy[off];
      if (MASK) g = relu_in[off] > 0 ? g : 0.0f;
      dx[off] = k * (g - a - (x[off] - mu) * b);
    }
  }
}

// Per-activation mode (N x D, one statistic per feature): a thread owns one
// feature, so warp accesses are coalesced along D; it walks the N rows twice.
__global__ void __launch_bounds__(128)
bn_bwd_peract_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                     const float* __restrict__ scale, const float* __restrict__ mean,
                     const float* __restrict__ invstd, float* __restrict__ dx,
                     float* __restrict__ dscale, float* __restrict__ dbias, int N, int D) {
  const int d = blockIdx.x * 128 + threadIdx.x;
  if (d >= D) return;
  const float mu = mean[d], r = invstd[d];
  float s_dy = 0.f, s_dyx = 0.f;
  for (int n = 0; n < N; ++n) {
    const float g = dy[static_cast<size_t>(n) * D + d];
    s_dy += g;
    s_dyx += g * (x[static_cast<size_t>(n) * D + d] - mu);
  }
  const float ds = s_dyx * r, inv_m = 1.0f / static_cast<float>(N);
  dscale[d] = ds;
  dbias[d] = s_dy;
  const float k = scale[d] * r, a = s_dy * inv_m, b = ds * r * inv_m;
  for (int n = 0; n < N; ++n) {
    const size_t off = static_cast<size_t>(n) * D + d;
    dx[off] = k * (dy[off] - a - (x[off] - mu) * b);
  }
}

template <bool MASK>
int bn_backward(const float* x, const float* dy, const float* relu_in, const float* scale,
                const float* mean, const float* invstd, float* dx, float* dscale,
                float* dbias, int N, int C, int HW, void* ws, size_t ws_bytes, void* stream) {
  if (N < 0 || C < 0 || HW < 0) return SGB_ERR_SIZE;
  if (N == 0 || C == 0 || HW == 0) return SGB_OK;
  if (!x || !dy || !scale || !mean || !invstd || !dx || !dscale || !dbias ||
      (MASK && !relu_in))
    return SGB_ERR_NULL;
  const long long per_channel = static_cast<long long>(N) * HW;
  if (per_channel > 0x7fffffffLL || C > 65535) return SGB_ERR_SIZE;
  cudaStream_t s = as_stream(stream);
  if (HW == 1 && !MASK) {
    bn_bwd_peract_kernel<<<static_cast<unsigned>(ceil_div(C, 128)), 128, 0, s>>>(
        x, dy, scale, mean, invstd, dx, dscale, dbias, N, C);
    return launch_status();
  }
  const int slices = bn_slices_for(per_channel, C, sm_count());
  if (!ws || ws_bytes < static_cast<size_t>(slices) * C * sizeof(float2) || !aligned16(ws))
    return SGB_ERR_WORKSPACE;
  float2* partial = static_cast<float2*>(ws);
  const bool vec = (HW % 4 == 0) && aligned16(x) && aligned16(dy) && aligned16(dx) &&
                   (!MASK || aligned16(relu_in));
  const BnShape sh{N, C, HW};
  const int total = static_cast<int>(vec ? per_channel / 4 : per_channel);
  const int per_slice = static_cast<int>(ceil_div(total, slices));
  const dim3 g1(slices, C), g2(static_cast<unsigned>(ceil_div(total, kBlock)), C);
  if (vec) {
    bn_bwd_reduce_kernel<true, MASK><<<g1, kBlock, 0, s>>>(x, dy, relu_in, mean, partial, sh, per_slice);
    bn_bwd_apply_kernel<true, MASK><<<g2, kBlock, 0, s>>>(x, dy, relu_in, scale, mean, invstd,
                                                          partial, slices, dx, dscale, dbias, sh);
  } else {
    bn_bwd_reduce_kernel<false, MASK><<<g1, kBlock, 0, s>>>(x, dy, relu_in, mean, partial, sh, per_slice);
    bn_bwd_apply_kernel<false, MASK><<<g2, kBlock, 0, s>>>(x, dy, relu_in, scale, mean, invstd,
                                                           partial, slices, dx, dscale, dbias, sh);
  }
  return launch_status();
}

}  // namespace
}  // namespace sgb

using namespace sgb;

extern "C" {

size_t sgb_bn_backward_workspace_bytes(int N, int C, int HW) {
  if (N <= 0 || C <= 0 || HW <= 0) return 0;
  return static_cast<size_t>(kMaxSlices) * C * sizeof(float2);
}

int sgb_bn_backward_f32(const float* x, const float* dy, const float* scale, const float* mean,
                        const float* invstd, float* dx, float* dscale, float* dbias, int N,
                        int C, int HW, void* ws, size_t ws_bytes, void* stream) {
  return bn_backward<false>(x, dy, nullptr, scale, mean, invstd, dx, dscale, dbias, N, C, HW,
                            ws, ws_bytes, stream);
}

int sgb_bn_relu_backward_f32(const float* x, const float* dy, const float* relu_in,
                             const float* scale, const float* mean, const float* invstd,
                             float* dx, float* dscale, float* dbias, int N, int C, int HW,
                             void* ws, size_t ws_bytes, void* stream) {
  return bn_backward<true>(x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias, N, C, HW,
                           ws, ws_bytes, stream);
}

}  // extern "C"
