// 2-D pooling (NCHW): max and average (divisor excludes padding), forward and
// backward.  Backward is written as a GATHER: every dx element visits the
// output windows that cover it, in raster order, and adds the gradients it is
// owed.  No atomics, so results are deterministic, and the order of additions
// equals that of a serial window-by-window scatter, which makes the result
// bit-identical to the CPU statement of the reference.
//
// Max backward credits, per window, the FIRST maximum in raster order (strict
// '>' while scanning, padding never wins).
#include <float.h>

#include "common.cuh"

namespace sgb {
namespace {

constexpr int kBlock = 256;

struct PoolShape {
  int N, C, H, W, OH, OW, kh, kw, ph, pw, sh, sw;
};

__device__ __forceinline__ void window(const PoolShape& p, int oh, int ow, int& h0, int& h1,
                                       int& w0, int& w1) {
  h0 = oh * p.sh - p.ph;
  w0 = ow * p.sw - p.pw;
  h1 = min(h0 + p.kh, p.H);
  w1 = min(w0 + p.kw, p.W);
  h0 = max(h0, 0);
  w0 = max(w0, 0);
}

// Range of output rows whose window contains input row h (same for columns).
__device__ __forceinline__ void covering(int h, int pad, int k, int stride, int out, int& lo,
                                         int& hi) {
  const int t = h + pad - k + 1;
  lo = t > 0 ? (t + stride - 1) / stride : 0;
  hi = min((h + pad) / stride, out - 1);
}

template <bool MAX>
__global__ void __launch_bounds__(kBlock)
pool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, PoolShape p, size_t total) {
  const size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x;
  if (i >= total) return;
  const int ow = static_cast<int>(i % p.OW);
  const int oh = static_cast<int>((i / p.OW) % p.OH);
  const size_t plane = i / (static_cast<size_t>(p.OW) * p.OH);
  const float* xp = x + plane * p.H * p.W;
  int h0, h1, w0, w1;
  window(p, oh, ow, h0, h1, w0, w1);
  if (MAX) {
    float best = -FLT_MAX;
    for (int h = h0; h < h1; ++h)
      for (int w = w0; w < w1; ++w) {
        const float v = xp[h * p.W + w];
        // a NaN in the window is the window's result (the reference's pooling
        // descriptor asks for CUDNN_PROPAGATE_NAN, src/model/operation/pooling.h:90):
        // the first NaN sticks, since nothing compares greater than it
        if (v > best || v != v) best = v;
      }
    y[i] = best;
  } else {
    float s = 0.f;
    for (int h = h0; h < h1; ++h)
      for (int w = w0; w < w1; ++w) s += xp[h * p.W + w];
    y[i] = s / static_cast<float>((h1 - h0) * (w1 - w0));
  }
}

// Max backward, one band of dx rows of one (n, c) plane per CTA.
//   phase 0: the x rows touched by the band's covering windows are staged in
//            shared memory with coalesced (128-bit when aligned) loads;
//   phase 1: every covering window finds its winner (first maximum in raster
//            order) in shared memory and parks the flat plane index;
//   phase 2: every dx element of the band gathers, in raster order, the dy of
//            the covering windows whose parked winner it is, and is stored
//            with a coalesced write.
// x is read from HBM once plus a one-window halo per band, dy and dx once.
struct BandPlan {
  int rows;        // dx rows per band
  int bands;       // bands per plane
  int max_xrows;   // x rows staged per band (upper bound)
  int max_orows;   // window rows per band (upper bound)
};

__global__ void __launch_bounds__(kBlock)
maxpool_bwd_band_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                        float* __restrict__ dx, PoolShape p, BandPlan bp) {
  extern __shared__ float smem[];
  float* xs = smem;                                            // max_xrows * W
  int* winner = reinterpret_cast<int*>(smem + bp.max_xrows * p.W);  // max_orows * OW
  const size_t plane = blockIdx.x;
  const int h_lo = blockIdx.y * bp.rows, h_hi = min(h_lo + bp.rows, p.H);  // dx rows [h_lo, h_hi)
  int o_lo, o_hi, unused;
  covering(h_lo, p.ph, p.kh, p.sh, p.OH, o_lo, unused);
  covering(h_hi - 1, p.ph, p.kh, p.sh, p.OH, unused, o_hi);    // window rows [o_lo, o_hi]
  const float* xp = x + plane * p.H * p.W;
  const float* gp = dy + plane * p.OH * p.OW;
  float* dp = dx + plane * p.H * p.W;
  if (o_hi >= o_lo) {
    const int xr_lo = max(o_lo * p.sh - p.ph, 0);
    const int xr_hi = min(o_hi * p.sh - p.ph + p.kh, p.H);     // x rows [xr_lo, xr_hi)
    const int nx = (xr_hi - xr_lo) * p.W;
    const float* src = xp + xr_lo * p.W;
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
      const int nv = nx >> 2;
      for (int v = threadIdx.x; v < nv; v += kBlock)
        reinterpret_cast<float4*>(xs)[v] = reinterpret_cast<const float4*>(src)[v];
      for (int i = (nv << 2) + threadIdx.x; i < nx; i += kBlock) xs[i] = src[i];
    } else {
      for (int i = threadIdx.x; i < nx; i += kBlock) xs[i] = src[i];
    }
    __syncthreads();
    const int nwin = (o_hi - o_lo + 1) * p.OW;
    for (int o = threadIdx.x; o < nwin; o += kBlock) {
      const int r = o / p.OW, ow = o - r * p.OW, oh = o_lo + r;
      int h0, h1, w0, w1;
      window(p, oh, ow, h0, h1, w0, w1);
      float best = -FLT_MAX;
      int bi = -1;
      for (int h = h0; h < h1; ++h) {
        const float* row = xs + (h - xr_lo) * p.W;
        for (int w = w0; w < w1; ++w) {
          const float v = row[w];
          if (v > best || (v != v && best == best)) {   // first maximum; a NaN wins and then sticks, as in cuDNN
            best = v;
            bi = h * p.W + w;
          }
        }
      }
      winner[o] = bi;
    }
  }
  __syncthreads();
  const int nin = (h_hi - h_lo) * p.W;
  for (int j = threadIdx.x; j < nin; j += kBlock) {
    const int r = j / p.W, w = j - r * p.W, h = h_lo + r;
    const int i = h * p.W + w;
    int oh_lo, oh_hi, ow_lo, ow_hi;
    covering(h, p.ph, p.kh, p.sh, p.OH, oh_lo, oh_hi);
    covering(w, p.pw, p.kw, p.sw, p.OW, ow_lo, ow_hi);
    float acc = 0.f;
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
      for (int ow = ow_lo; ow <= ow_hi; ++ow)
        if (winner[(oh - o_lo) * p.OW + ow] == i) acc += gp[oh * p.OW + ow];
    dp[i] = acc;
  }
}

// Same scheme with the geometry (square kernel K, stride S, padding P) known
// at compile time: window loops unroll, the divisions by the stride become
// shifts, dy rows are staged in shared memory as well, and every thread
// produces four consecutive dx values of one row (one 128-bit store).  This is
// the form the ResNet stem (3x3 / 2 / 1) and the small CNN (2x2 / 2 / 0) hit;
// it needs W % 4 == 0.  About 60 instructions per dx element instead of ~200.
template <int K, int S, int P>
__global__ void __launch_bounds__(kBlock)
maxpool_bwd_band_fast_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                             float* __restrict__ dx, PoolShape p, BandPlan bp) {
  extern __shared__ float smem[];
  float* xs = smem;
  int* winner = reinterpret_cast<int*>(xs + bp.max_xrows * p.W);
  float* gs = reinterpret_cast<float*>(winner + bp.max_orows * p.OW);
  const size_t plane = blockIdx.x;
  const int H = p.H, W = p.W, OH = p.OH, OW = p.OW;
  const int h_lo = blockIdx.y * bp.rows, h_hi = min(h_lo + bp.rows, H);
  const int t_lo = h_lo + P - K + 1;
  const int o_lo = t_lo > 0 ? (t_lo + S - 1) / S : 0;
  const int o_hi = min((h_hi - 1 + P) / S, OH - 1);
  const float* xp = x + plane * H * W;
  const float* gp = dy + plane * OH * OW;
  float* dp = dx + plane * H * W;
  const int xr_lo = max(o_lo * S - P, 0);
  if (o_hi >= o_lo) {
    const int xr_hi = min(o_hi * S - P + K, H);
    const int nv = ((xr_hi - xr_lo) * W) >> 2;                 // W % 4 == 0
    const float4* src = reinterpret_cast<const float4*>(xp + xr_lo * W);
    for (int v = threadIdx.x; v < nv; v += kBlock) reinterpret_cast<float4*>(xs)[v] = src[v];
    const int nwin = (o_hi - o_lo + 1) * OW;
    const float* gsrc = gp + o_lo * OW;
    for (int o = threadIdx.x; o < nwin; o += kBlock) gs[o] = gsrc[o];
    __syncthreads();
    for (int o = threadIdx.x; o < nwin; o += kBlock) {
      const int r = o / OW, ow = o - r * OW, oh = o_lo + r;
      float best = -FLT_MAX;
      int bi = -1;
#pragma unroll
      for (int i = 0; i < K; ++i) {
        const int h = oh * S - P + i;
        if (h < 0 || h >= H) continue;
        const float* row = xs + (h - xr_lo) * W;
#pragma unroll
        for (int j = 0; j < K; ++j) {
          const int w = ow * S - P + j;
          if (w < 0 || w >= W) continue;
          const float v = row[w];
          if (v > best || (v != v && best == best)) {   // first maximum; a NaN wins and then sticks, as in cuDNN
            best = v;
            bi = h * W + w;
          }
        }
      }
      winner[o] = bi;
    }
  }
  __syncthreads();
  constexpr int kCover = (K + S - 1) / S;                       // windows covering one row/column
  const int w4 = W >> 2, nq = (h_hi - h_lo) * w4;
  for (int q = threadIdx.x; q < nq; q += kBlock) {
    const int r = q / w4, c4 = q - r * w4, h = h_lo + r;
    const int th = h + P - K + 1;
    const int oh_lo = th > 0 ? (th + S - 1) / S : 0;
    const int oh_hi = min((h + P) / S, OH - 1);
    float out[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int w = 4 * c4 + e, i = h * W + w;
      const int tw = w + P - K + 1;
      const int ow_lo = tw > 0 ? (tw + S - 1) / S : 0;
      const int ow_hi = min((w + P) / S, OW - 1);
      float acc = 0.f;
#pragma unroll
      for (int a = 0; a < kCover; ++a) {
        const int oh = oh_lo + a;
        if (oh > oh_hi) break;
#pragma unroll
        for (int b = 0; b < kCover; ++b) {
          const int ow = ow_lo + b;
          if (ow > ow_hi) break;
          const int widx = (oh - o_lo) * OW + ow;
          if (winner[widx] == i) acc += gs[widx];
        }
      }
      out[e] = acc;
    }
    *reinterpret_cast<float4*>(dp + h * W + 4 * c4) = make_float4(out[0], out[1], out[2], out[3]);
  }
}

// 3x3 window, stride 2, padding 1 on even H and W % 4 == 0 (the ResNet stem):
// the general scheme above with everything that can be decided at compile time
// decided.  The staged x band carries a -FLT_MAX column on the left and, at the
// top of the plane, a -FLT_MAX row, so the nine reads of a window need no
// bounds tests; every thread then produces a 2 x 4 patch of dx from six parked
// winners (two window rows x three window columns), whose raster-order sums
// are written out explicitly.  ~30 instructions per dx element.
struct StemPlan {
  int rows;     // dx rows per band (even)
  int bands;
};

// WC: plane width known at compile time (0 = use the run-time value); with a
// constant width the row / column splits below compile to multiply-shift
// sequences instead of integer divisions, a quarter of the kernel's instructions.
template <int WC>
__global__ void __launch_bounds__(kBlock)
maxpool_bwd_k3s2p1_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                          float* __restrict__ dx, int H, int W_rt, int OH, int OW_rt, int rows) {
  extern __shared__ float smem[];
  const int W = WC ? WC : W_rt;
  const int OW = WC ? WC / 2 : OW_rt;
  const int pitch = W + 4;                       // xs[r][4 + c] = x[xr0 + r][c], xs[r][3] = -FLT_MAX
  const int wp = OW + 1;                         // winner / dy pitch (one never-matching pad column)
  const int h_lo = blockIdx.y * rows, h_hi = min(h_lo + rows, H);
  const int o_lo = h_lo >> 1, o_hi = min(h_hi >> 1, OH - 1);     // window rows [o_lo, o_hi]
  const int norow = o_hi - o_lo + 1;
  const int xr0 = 2 * o_lo - 1;                                 // may be -1
  const int xr1 = min(2 * o_hi + 2, H);                         // x rows [xr0, xr1)
  const int nxr = xr1 - xr0;
  float* xs = smem;
  int* winner = reinterpret_cast<int*>(xs + (rows + 3) * pitch);
  float* gs = reinterpret_cast<float*>(winner + ((rows >> 1) + 2) * wp);
  const size_t plane = blockIdx.x;
  const float* xp = x + plane * H * W;
  const float* gp = dy + plane * OH * OW;
  float* dp = dx + plane * H * W;

  const int w4 = W >> 2;
  for (int v = threadIdx.x; v < nxr * w4; v += kBlock) {
    const int r = v / w4, c4 = v - r * w4, xr = xr0 + r;
    float4 val = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
    if (xr >= 0) val = *reinterpret_cast<const float4*>(xp + xr * W + 4 * c4);
    *reinterpret_cast<float4*>(xs + r * pitch + 4 + 4 * c4) = val;
  }
  for (int r = threadIdx.x; r < nxr; r += kBlock) xs[r * pitch + 3] = -FLT_MAX;
  // dy rows of the band's windows, plus a pad row / column of winners that match nothing
  for (int o = threadIdx.x; o < (norow + 1) * wp; o += kBlock) {
    const int r = o / wp, c = o - r * wp;
    const bool real = r < norow && c < OW;
    gs[o] = real ? gp[(o_lo + r) * OW + c] : 0.0f;
    if (!real) winner[o] = -2;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < norow * OW; o += kBlock) {
    const int r = o / OW, ow = o - r * OW;
    const float* win = xs + (2 * r) * pitch + 2 * ow + 3;        // top-left cell of the window
    const int g0 = (2 * (o_lo + r) - 1) * W + 2 * ow - 1;        // its flat plane index
    float best = -FLT_MAX;
    int bi = -1;
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const float v = win[i * pitch + j];
        if (v > best || (v != v && best == best)) {   // first maximum; a NaN wins and then sticks, as in cuDNN
          best = v;
          bi = g0 + i * W + j;
        }
      }
    winner[r * wp + ow] = bi;
  }
  __syncthreads();
  const int npatch = ((h_hi - h_lo) >> 1) * w4;
  for (int t = threadIdx.x; t < npatch; t += kBlock) {
    const int m = t / w4, q = t - m * w4;
    const int* w0 = winner + m * wp + 2 * q;       // windows (m, 2q .. 2q+2)
    const int* w1 = w0 + wp;                        // windows (m+1, ...)
    const float* g0 = gs + m * wp + 2 * q;
    const float* g1 = g0 + wp;
    const int a0 = w0[0], a1 = w0[1], a2 = w0[2], b0 = w1[0], b1 = w1[1], b2 = w1[2];
    const float ga0 = g0[0], ga1 = g0[1], ga2 = g0[2], gb0 = g1[0], gb1 = g1[1], gb2 = g1[2];
    const int h = h_lo + 2 * m;
    const int i0 = h * W + 4 * q, i1 = i0 + W;      // flat indices of the patch's two rows
#define PICK(wv, gv, idx) ((wv) == (idx) ? (gv) : 0.0f)
    float4 top, bot;
    top.x = 0.0f + PICK(a0, ga0, i0);
    top.y = (0.0f + PICK(a0, ga0, i0 + 1)) + PICK(a1, ga1, i0 + 1);
    top.z = 0.0f + PICK(a1, ga1, i0 + 2);
    top.w = (0.0f + PICK(a1, ga1, i0 + 3)) + PICK(a2, ga2, i0 + 3);
    bot.x = (0.0f + PICK(a0, ga0, i1)) + PICK(b0, gb0, i1);
    bot.y = (((0.0f + PICK(a0, ga0, i1 + 1)) + PICK(a1, ga1, i1 + 1)) + PICK(b0, gb0, i1 + 1)) +
            PICK(b1, gb1, i1 + 1);
    bot.z = (0.0f + PICK(a1, ga1, i1 + 2)) + PICK(b1, gb1, i1 + 2);
    bot.w = (((0.0f + PICK(a1, ga1, i1 + 3)) + PICK(a2, ga2, i1 + 3)) + PICK(b1, gb1, i1 + 3)) +
            PICK(b2, gb2, i1 + 3);
#undef PICK
    *reinterpret_cast<float4*>(dp + i0) = top;
    *reinterpret_cast<float4*>(dp + i1) = bot;
  }
}

// ------------------------------------------------ arg-max forward partner
// Max-pool forward that also records, per window, WHERE its (first, in raster
// order) maximum sits: one byte, row offset in the high nibble and column
// offset in the low nibble, both relative to the window's unclipped top-left
// corner (oh*sh - ph, ow*sw - pw).  With that record the backward pass needs
// neither x nor y: it reads dy and one byte per window.
__global__ void __launch_bounds__(kBlock)
maxpool_fwd_argmax_kernel(const float* __restrict__ x, float* __restrict__ y,
                          unsigned char* __restrict__ arg, PoolShape p, size_t total) {
  const size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x;
  if (i >= total) return;
  const int ow = static_cast<int>(i % p.OW);
  const int oh = static_cast<int>((i / p.OW) % p.OH);
  const size_t plane = i / (static_cast<size_t>(p.OW) * p.OH);
  const float* xp = x + plane * p.H * p.W;
  int h0, h1, w0, w1;
  window(p, oh, ow, h0, h1, w0, w1);
  const int hs = oh * p.sh - p.ph, ws = ow * p.sw - p.pw;
  float best = -FLT_MAX;
  int code = 0xff;                                  // matches no cell (empty or all -FLT_MAX window)
  for (int h = h0; h < h1; ++h)
    for (int w = w0; w < w1; ++w) {
      const float v = xp[h * p.W + w];
      if (v > best || (v != v && best == best)) {   // first maximum, or the first NaN (which then sticks)
        best = v;
        code = ((h - hs) << 4) | (w - ws);
      }
    }
  y[i] = best;
  arg[i] = static_cast<unsigned char>(code);
}

// Backward from the record, any geometry: one dx element per thread gathers,
// in raster order of the windows, the dy of every covering window whose
// record points at it.
__global__ void __launch_bounds__(kBlock)
maxpool_bwd_argmax_kernel(const float* __restrict__ dy, const unsigned char* __restrict__ arg,
                          float* __restrict__ dx, PoolShape p, size_t total) {
  const size_t i = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x;
  if (i >= total) return;
  const int w = static_cast<int>(i % p.W);
  const int h = static_cast<int>((i / p.W) % p.H);
  const size_t plane = i / (static_cast<size_t>(p.W) * p.H);
  const float* gp = dy + plane * p.OH * p.OW;
  const unsigned char* ap = arg + plane * p.OH * p.OW;
  int oh_lo, oh_hi, ow_lo, ow_hi;
  covering(h, p.ph, p.kh, p.sh, p.OH, oh_lo, oh_hi);
  covering(w, p.pw, p.kw, p.sw, p.OW, ow_lo, ow_hi);
  float acc = 0.f;
  for (int oh = oh_lo; oh <= oh_hi; ++oh)
    for (int ow = ow_lo; ow <= ow_hi; ++ow) {
      const int code = ap[oh * p.OW + ow];
      const int wh = oh * p.sh - p.ph + (code >> 4), ww = ow * p.sw - p.pw + (code & 15);
      if (code != 0xff && wh == h && ww == w) acc += gp[oh * p.OW + ow];
    }
  dx[i] = acc;
}

// Backward from the record for 3x3 / stride 2 / pad 1 (ResNet stem): the same
// band / 2x4-patch scheme as maxpool_bwd_k3s2p1_kernel without its x staging
// and winner search - the parked winners come straight from the record.
template <int WC>
__global__ void __launch_bounds__(kBlock)
maxpool_bwd_argmax_k3s2p1_kernel(const float* __restrict__ dy, const unsigned char* __restrict__ arg,
                                 float* __restrict__ dx, int H, int W_rt, int OH, int OW_rt, int rows) {
  extern __shared__ float smem[];
  const int W = WC ? WC : W_rt;
  const int OW = WC ? WC / 2 : OW_rt;
  const int wp = OW + 1;                         // winner / dy pitch (one never-matching pad column)
  const int h_lo = blockIdx.y * rows, h_hi = min(h_lo + rows, H);
  const int o_lo = h_lo >> 1, o_hi = min(h_hi >> 1, OH - 1);     // window rows [o_lo, o_hi]
  const int norow = o_hi - o_lo + 1;
  int* winner = reinterpret_cast<int*>(smem);
  float* gs = reinterpret_cast<float*>(winner + ((rows >> 1) + 2) * wp);
  const size_t plane = blockIdx.x;
  const float* gp = dy + plane * OH * OW;
  const unsigned char* ap = arg + plane * OH * OW;
  float* dp = dx + plane * H * W;
  for (int o = threadIdx.x; o < (norow + 1) * wp; o += kBlock) {
    const int r = o / wp, c = o - r * wp;
    const bool real = r < norow && c < OW;
    float g = 0.0f;
    int win = -2;
    if (real) {
      const int oh = o_lo + r;
      g = gp[oh * OW + c];
      const int code = ap[oh * OW + c];
      if (code != 0xff) win = (2 * oh - 1 + (code >> 4)) * W + 2 * c - 1 + (code & 15);
    }
    gs[o] = g;
    winner[o] = win;
  }
  __syncthreads();
  const int w4 = W >> 2;
  const int npatch = ((h_hi - h_lo) >> 1) * w4;
  for (int t = threadIdx.x; t < npatch; t += kBlock) {
    const int m = t / w4, q = t - m * w4;
    const int* w0 = winner + m * wp + 2 * q;       // windows (m, 2q .. 2q+2)
    const int* w1 = w0 + wp;                        // windows (m+1, ...)
    const float* g0 = gs + m * wp + 2 * q;
    const float* g1 = g0 + wp;
    const int a0 = w0[0], a1 = w0[1], a2 = w0[2], b0 = w1[0], b1 = w1[1], b2 = w1[2];
    const float ga0 = g0[0], ga1 = g0[1], ga2 = g0[2], gb0 = g1[0], gb1 = g1[1], gb2 = g1[2];
    const int h = h_lo + 2 * m;
    const int i0 = h * W + 4 * q, i1 = i0 + W;      // flat indices of the patch's two rows
#define PICK(wv, gv, idx) ((wv) == (idx) ? (gv) : 0.0f)
    float4 top, bot;
    top.x = 0.0f + PICK(a0, ga0, i0);
    top.y = (0.0f + PICK(a0, ga0, i0 + 1)) + PICK(a1, ga1, i0 + 1);
    top.z = 0.0f + PICK(a1, ga1, i0 + 2);
    top.w = (0.0f + PICK(a1, ga1, i0 + 3)) + PICK(a2, ga2, i0 + 3);
    bot.x = (0.0f + PICK(a0, ga0, i1)) + PICK(b0, gb0, i1);
    bot.y = (((0.0f + PICK(a0, ga0, i1 + 1)) + PICK(a1, ga1, i1 + 1)) + PICK(b0, gb0, i1 + 1)) +
            PICK(b1, gb1, i1 + 1);
    bot.z = (0.0f + PICK(a1, ga1, i1 + 2)) + PICK(b1, gb1, i1 + 2);
    bot.w = (((0.0f + PICK(a1, ga1, i1 + 3)) + PICK(a2, ga2, i1 + 3)) + PICK(b1, gb1, i1 + 3)) +
            PICK(b2, gb2, i1 + 3);
#undef PICK
    *reinterpret_cast<float4*>(dp + i0) = top;
    *reinterpret_cast<float4*>(dp + i1) = bot;
  }
}

// Band height: the largest power-of-two-ish row count whose staging fits
// `budget` bytes of shared memory; 0 rows means even one row does not fit.
BandPlan plan_bands(const PoolShape& p, size_t budget) {
  BandPlan bp{0, 0, 0, 0};
  for (int rows = p.H; rows >= 1; rows = (rows > 64 ? (rows + 1) / 2 : rows - 1)) {
    // windows covering `rows` consecutive dx rows, and the x rows they touch
    const int orows = min((rows + p.kh - 2) / p.sh + 2, p.OH);
    const int xrows = min((orows - 1) * p.sh + p.kh, p.H);
    const size_t bytes = (static_cast<size_t>(xrows) * p.W + 2 * static_cast<size_t>(orows) * p.OW) * 4;
    if (bytes <= budget) {
      bp.rows = rows;
      bp.bands = (p.H + rows - 1) / rows;
      bp.max_xrows = xrows;
      bp.max_orows = orows;
      return bp;
    }
  }
  return bp;
}

// Fallback for planes whose winner table does not fit shared memory: every dx
// element re-derives the winner of each covering window from x.
__global__ void __launch_bounds__(kBlock)
maxpool_bwd_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                   float* __restrict__ dx, PoolShape p) {
  const size_t plane = blockIdx.x;
  const int i = blockIdx.y * kBlock + threadIdx.x;
  if (i >= p.H * p.W) return;
  const int h = i / p.W, w = i - h * p.W;
  const float* xp = x + plane * p.H * p.W;
  const float* gp = dy + plane * p.OH * p.OW;
  const float mine = xp[i];
  int oh_lo, oh_hi, ow_lo, ow_hi;
  covering(h, p.ph, p.kh, p.sh, p.OH, oh_lo, oh_hi);
  covering(w, p.pw, p.kw, p.sw, p.OW, ow_lo, ow_hi);
  float acc = 0.f;
  for (int oh = oh_lo; oh <= oh_hi; ++oh)
    for (int ow = ow_lo; ow <= ow_hi; ++ow) {
      int h0, h1, w0, w1;
      window(p, oh, ow, h0, h1, w0, w1);
      // (h, w) wins this window iff nothing before it (raster order) is >= it
      // and nothing after it is > it, and it beats the -FLT_MAX seed.
      bool win = mine > -FLT_MAX;
      for (int hh = h0; hh < h1 && win; ++hh)
        for (int ww = w0; ww < w1; ++ww) {
          const float v = xp[hh * p.W + ww];
          const bool before = hh < h || (hh == h && ww < w);
          if (before ? (v >= mine) : (v > mine)) {
            win = false;
            break;
          }
        }
      if (win) acc += gp[oh * p.OW + ow];
    }
  dx[plane * p.H * p.W + i] = acc;
}

// Average backward: one thread per dx element over the flattened tensor
// (chunks of < 2^31 elements so the index arithmetic stays 32-bit).
__global__ void __launch_bounds__(kBlock)
avgpool_bwd_kernel(const float* __restrict__ dy, float* __restrict__ dx, PoolShape p,
                   unsigned total) {
  const unsigned i = blockIdx.x * static_cast<unsigned>(kBlock) + threadIdx.x;
  if (i >= total) return;
  const unsigned hw = static_cast<unsigned>(p.H * p.W);
  const unsigned plane = i / hw, r = i - plane * hw;
  const int h = static_cast<int>(r / static_cast<unsigned>(p.W)), w = static_cast<int>(r) - h * p.W;
  const float* gp = dy + static_cast<size_t>(plane) * p.OH * p.OW;
  int oh_lo, oh_hi, ow_lo, ow_hi;
  covering(h, p.ph, p.kh, p.sh, p.OH, oh_lo, oh_hi);
  covering(w, p.pw, p.kw, p.sw, p.OW, ow_lo, ow_hi);
  float acc = 0.f;
  for (int oh = oh_lo; oh <= oh_hi; ++oh)
    for (int ow = ow_lo; ow <= ow_hi; ++ow) {
      int h0, h1, w0, w1;
      window(p, oh, ow, h0, h1, w0, w1);
      acc += gp[oh * p.OW + ow] / static_cast<float>((h1 - h0) * (w1 - w0));
    }
  dx[i] = acc;
}

// Global average pooling (one window = the whole plane, no padding): every dx
// element of a plane is dy[plane] / (H*W).  Four consecutive elements per
// thread, one 128-bit store; the plane index advances without extra divisions.
__global__ void __launch_bounds__(kBlock)
avgpool_bwd_global_kernel(const float* __restrict__ dy, float* __restrict__ dx, unsigned hw,
                          unsigned total4) {
  const unsigned v = blockIdx.x * static_cast<unsigned>(kBlock) + threadIdx.x;
  if (v >= total4) return;
  const unsigned i = 4u * v;
  unsigned plane = i / hw, r = i - plane * hw;
  const float inv = static_cast<float>(hw);
  float out[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    out[e] = dy[plane] / inv;
    if (++r == hw) {
      r = 0;
      ++plane;
    }
  }
  *reinterpret_cast<float4*>(dx + i) = make_float4(out[0], out[1], out[2], out[3]);
}

int make_shape(PoolShape& p, int N, int C, int H, int W, int kh, int kw, int ph, int pw, int sh,
               int sw) {
  if (N < 0 || C < 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || ph < 0 || pw < 0 || sh <= 0 ||
      sw <= 0)
    return SGB_ERR_SIZE;
  if (ph >= kh || pw >= kw) return SGB_ERR_SIZE;  // a window must touch the image
  if (H + 2 * ph < kh || W + 2 * pw < kw) return SGB_ERR_SIZE;
  p = PoolShape{N, C, H, W, (H + 2 * ph - kh) / sh + 1, (W + 2 * pw - kw) / sw + 1,
                kh, kw, ph, pw, sh, sw};
  return SGB_OK;
}

unsigned blocks_for(size_t total) { return static_cast<unsigned>(ceil_div(total, kBlock)); }

}  // namespace
}  // namespace sgb

using namespace sgb;

extern "C" {

int sgb_pool_out_size(int in, int kernel, int pad, int stride) {
  if (stride <= 0) return 1;
  return (in + 2 * pad - kernel) / stride + 1;
}

#define POOL_PROLOGUE(OUT_IS_Y)                                                        \
  PoolShape p;                                                                         \
  int st = make_shape(p, N, C, H, W, kh, kw, ph, pw, sh, sw);                          \
  if (st != SGB_OK) return st;                                                         \
  const size_t in_total = static_cast<size_t>(N) * C * H * W;                          \
  const size_t out_total = static_cast<size_t>(N) * C * p.OH * p.OW;                   \
  (void)in_total; (void)out_total;                                                     \
  if (in_total == 0) return SGB_OK;                                                    \
  if (ceil_div(in_total, kBlock) > 0x7fffffffu) return SGB_ERR_SIZE;

int sgb_maxpool_forward_f32(const float* x, float* y, int N, int C, int H, int W, int kh, int kw,
                            int ph, int pw, int sh, int sw, void* stream) {
  POOL_PROLOGUE(1)
  if (!x || !y) return SGB_ERR_NULL;
  pool_fwd_kernel<true><<<blocks_for(out_total), kBlock, 0, as_stream(stream)>>>(x, y, p, out_total);
  return launch_status();
}

int sgb_avgpool_forward_f32(const float* x, float* y, int N, int C, int H, int W, int kh, int kw,
                            int ph, int pw, int sh, int sw, void* stream) {
  POOL_PROLOGUE(1)
  if (!x || !y) return SGB_ERR_NULL;
  pool_fwd_kernel<false><<<blocks_for(out_total), kBlock, 0, as_stream(stream)>>>(x, y, p, out_total);
  return launch_status();
}

int sgb_maxpool_backward_f32(const float* x, const float* y, const float* dy, float* dx, int N,
                             int C, int H, int W, int kh, int kw, int ph, int pw, int sh, int sw,
                             void* stream) {
  (void)y;  // the winner is recomputed from x; y is accepted for interface parity
  POOL_PROLOGUE(0)
  if (!x || !dy || !dx) return SGB_ERR_NULL;
  const size_t planes = static_cast<size_t>(N) * C;
  if (planes > 0x7fffffffu || static_cast<long long>(H) * W > 0x7fffffffLL) return SGB_ERR_SIZE;
  const BandPlan bp = plan_bands(p, 24 * 1024);
  if (bp.rows > 0 && bp.bands <= 65535) {
    const size_t smem = (static_cast<size_t>(bp.max_xrows) * W +
                         2 * static_cast<size_t>(bp.max_orows) * p.OW) * sizeof(float);
    const dim3 grid(static_cast<unsigned>(planes), bp.bands);
    cudaStream_t s = as_stream(stream);
    const bool square = kh == kw && sh == sw && ph == pw && W % 4 == 0 && aligned16(x) && aligned16(dx);
    if (square && kh == 3 && sh == 2 && ph == 1 && H % 2 == 0 && H >= 2) {
      const int nb = (H + 31) / 32;
      int rows = (H + nb - 1) / nb;
      rows += rows & 1;
      const int nbands = (H + rows - 1) / rows;
      const size_t bytes = (static_cast<size_t>(rows + 3) * (W + 4) +
                            2 * static_cast<size_t>((rows >> 1) + 2) * (p.OW + 1)) * sizeof(float);
      if (bytes <= 48 * 1024 && nbands <= 65535) {
        const dim3 g(static_cast<unsigned>(planes), nbands);
#define SGB_STEM_W(WW)                                                                              \
  if (W == WW && p.OW == WW / 2) {                                                                  \
    maxpool_bwd_k3s2p1_kernel<WW><<<g, kBlock, bytes, s>>>(x, dy, dx, H, W, p.OH, p.OW, rows);      \
    return launch_status();                                                                         \
  }
        SGB_STEM_W(112)
        SGB_STEM_W(56)
        SGB_STEM_W(32)
#undef SGB_STEM_W
        maxpool_bwd_k3s2p1_kernel<0><<<g, kBlock, bytes, s>>>(x, dy, dx, H, W, p.OH, p.OW, rows);
        return launch_status();
      }
    }
#define SGB_POOL_FAST(KK, SS, PP)                                                       \
  if (square && kh == KK && sh == SS && ph == PP) {                                     \
    maxpool_bwd_band_fast_kernel<KK, SS, PP><<<grid, kBlock, smem, s>>>(x, dy, dx, p, bp); \
    return launch_status();                                                             \
  }
    SGB_POOL_FAST(3, 2, 1)
    SGB_POOL_FAST(2, 2, 0)
    SGB_POOL_FAST(3, 2, 0)
    SGB_POOL_FAST(3, 1, 1)
    SGB_POOL_FAST(2, 1, 0)
#undef SGB_POOL_FAST
    maxpool_bwd_band_kernel<<<grid, kBlock, smem, s>>>(x, dy, dx, p, bp);
  } else {
    const unsigned by = blocks_for(static_cast<size_t>(H) * W);
    if (by > 65535) return SGB_ERR_SIZE;
    maxpool_bwd_kernel<<<dim3(static_cast<unsigned>(planes), by), kBlock, 0, as_stream(stream)>>>(
        x, dy, dx, p);
  }
  return launch_status();
}

int sgb_maxpool_forward_argmax_f32(const float* x, float* y, unsigned char* argmax, int N, int C, int H,
                                   int W, int kh, int kw, int ph, int pw, int sh, int sw, void* stream) {
  POOL_PROLOGUE(1)
  if (!x || !y || !argmax) return SGB_ERR_NULL;
  if (kh > 15 || kw > 15) return SGB_ERR_UNSUPPORTED;           // offsets are stored in nibbles; 15|15 is "none"
  maxpool_fwd_argmax_kernel<<<blocks_for(out_total), kBlock, 0, as_stream(stream)>>>(x, y, argmax, p, out_total);
  return launch_status();
}

int sgb_maxpool_backward_argmax_f32(const float* dy, const unsigned char* argmax, float* dx, int N, int C,
                                    int H, int W, int kh, int kw, int ph, int pw, int sh, int sw,
                                    void* stream) {
  POOL_PROLOGUE(0)
  if (!dy || !argmax || !dx) return SGB_ERR_NULL;
  if (kh > 15 || kw > 15) return SGB_ERR_UNSUPPORTED;
  const size_t planes = static_cast<size_t>(N) * C;
  cudaStream_t s = as_stream(stream);
  if (kh == 3 && kw == 3 && sh == 2 && sw == 2 && ph == 1 && pw == 1 && W % 4 == 0 && H % 2 == 0 && H >= 2 &&
      aligned16(dx) && planes <= 0x7fffffffu && static_cast<long long>(H) * W <= 0x7fffffffLL) {
    const int nb = (H + 31) / 32;
    int rows = (H + nb - 1) / nb;
    rows += rows & 1;
    const int nbands = (H + rows - 1) / rows;
    const size_t bytes = 2 * static_cast<size_t>((rows >> 1) + 2) * (p.OW + 1) * sizeof(float);
    if (bytes <= 48 * 1024 && nbands <= 65535) {
      const dim3 g(static_cast<unsigned>(planes), nbands);
#define SGB_STEM_W(WW)                                                                                  \
  if (W == WW && p.OW == WW / 2) {                                                                      \
    maxpool_bwd_argmax_k3s2p1_kernel<WW><<<g, kBlock, bytes, s>>>(dy, argmax, dx, H, W, p.OH, p.OW, rows); \
    return launch_status();                                                                             \
  }
      SGB_STEM_W(112)
      SGB_STEM_W(56)
      SGB_STEM_W(32)
#undef SGB_STEM_W
      maxpool_bwd_argmax_k3s2p1_kernel<0><<<g, kBlock, bytes, s>>>(dy, argmax, dx, H, W, p.OH, p.OW, rows);
      return launch_status();
    }
  }
  maxpool_bwd_argmax_kernel<<<blocks_for(in_total), kBlock, 0, s>>>(dy, argmax, dx, p, in_total);
  return launch_status();
}

int sgb_avgpool_backward_f32(const float* dy, float* dx, int N, int C, int H, int W, int kh,
                             int kw, int ph, int pw, int sh, int sw, void* stream) {
  POOL_PROLOGUE(0)
  if (!dy || !dx) return SGB_ERR_NULL;
  const size_t planes = static_cast<size_t>(N) * C;
  if (static_cast<long long>(H) * W > 0x7fffffffLL) return SGB_ERR_SIZE;
  if (p.OH == 1 && p.OW == 1 && ph == 0 && pw == 0 && kh == H && kw == W && aligned16(dx) &&
      in_total % 4 == 0 && in_total < 0x7fffffffu) {
    const unsigned total4 = static_cast<unsigned>(in_total / 4);
    avgpool_bwd_global_kernel<<<blocks_for(total4), kBlock, 0, as_stream(stream)>>>(
        dy, dx, static_cast<unsigned>(H * W), total4);
    return launch_status();
  }
  // whole planes per launch, each launch below 2^31 elements
  const size_t hw = static_cast<size_t>(H) * W;
  const size_t planes_per_launch = (0x7fffffffu - kBlock) / hw;
  if (planes_per_launch == 0) return SGB_ERR_SIZE;
  for (size_t p0 = 0; p0 < planes; p0 += planes_per_launch) {
    const size_t np = planes - p0 < planes_per_launch ? planes - p0 : planes_per_launch;
    const unsigned total = static_cast<unsigned>(np * hw);
    avgpool_bwd_kernel<<<blocks_for(total), kBlock, 0, as_stream(stream)>>>(
        dy + p0 * p.OH * p.OW, dx + p0 * hw, p, total);
  }
  return launch_status();
}

}  // extern "C"
