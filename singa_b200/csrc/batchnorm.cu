// Batch-normalisation backward (training mode) with saved mean and saved
// inverse standard deviation:
//   dbias[c]  = sum dy
//   dscale[c] = sum dy * (x - mean[c]) * invstd[c]
//   dx        = scale[c] * invstd[c] *
//               (dy - dbias[c]/M - (x - mean[c]) * invstd[c] * dscale[c] / M)
// M = N*H*W (spatial mode, NCHW) or N (per-activation mode, N x D).
//
// Single-pass scheme (12 bytes of HBM traffic per element), used whenever one
// channel's x and dy (N*H*W*8 bytes) fit the shared memory of a thread-block
// cluster of at most 8 CTAs: the cluster stages its channel in shared memory
// with 16-byte asynchronous copies (cp.async, no register staging), every CTA
// reduces its share with warp shuffles, the CTAs exchange their two partial
// sums through distributed shared memory, and dx is computed from the staged
// copy.  Shares are sized so that two to four CTAs are resident per SM and
// the load phase of one overlaps the store phase of another.
//
// Channels too large for a cluster (e.g. 32 x 112 x 112) are also done in one
// pass, by the streaming kernel of bn_stream.cu: persistent small CTAs take
// 50 KB items of a channel from a ticket counter and meet through counters in
// global memory.
//
// Two-pass scheme, 20 bytes of HBM traffic per element when the tensor does
// not fit L2; the fallback for planes that are not a multiple of four floats,
// misaligned operands, more than 4096 channels, and the entry point without
// workspace:
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
#include <cooperative_groups.h>
#include <stdlib.h>

#include <atomic>

#include "bn_stream.cuh"
#include "bulk_copy.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace sgb {
namespace {

constexpr int kBlock = 256;
constexpr int kMaxSlices = 64;

// Opts a kernel in to more than 48 KB of dynamic shared memory (and, for the
// cluster kernels, to non-portable cluster sizes) once per device: the
// attribute sticks to the function in that device's context, so later
// launches - including launches under stream capture - issue no attribute
// call.  `done` is one flag per device ordinal; ordinals beyond the table are
// set every time.  Racing first calls from two host threads both set the
// same attribute, which is harmless.
template <typename K>
int opt_in_once(K kernel, std::atomic<bool>* done, bool cluster) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && done[dev].load(std::memory_order_acquire)) return SGB_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  if (e != cudaSuccess) return note_cuda_error(e);
  if (cluster) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return note_cuda_error(e);
  }
  if (tracked) done[dev].store(true, std::memory_order_release);
  return SGB_OK;
}

struct BnShape {
  int N, C, HW;
};

// Walks the units u0 + tid, u0 + tid + T, ... of a share and keeps the
// (plane n, position q) decomposition up to date without a division per step.
struct UnitWalk {
  int n, q, dn, dq, hwu;
  __device__ __forceinline__ UnitWalk(int u, int step, int hwu_) : hwu(hwu_) {
    n = u / hwu_;
    q = u - n * hwu_;
    dn = step / hwu_;
    dq = step - dn * hwu_;
  }
  __device__ __forceinline__ void next() {
    n += dn;
    q += dq;
    if (q >= hwu) {
      q -= hwu;
      ++n;
    }
  }
};

// How the fused ReLU backward learns which gradients to keep.  MASK 0: no ReLU.
// MASK 1: from the ReLU's stored input (keep where it is > 0).  MASK 2: from the
// forward partner's record, one bit per element in element order (bit i & 7 of
// byte i >> 3; 1 = the input was > 0), passed through the same pointer.
// `off` is the element offset; for the 4-wide forms it is a multiple of 4.
template <int MASK>
__device__ __forceinline__ unsigned keep4(const float* relu_in, size_t off) {
  if (MASK == 2) {
    const unsigned char b = reinterpret_cast<const unsigned char*>(relu_in)[off >> 3];
    return (b >> (off & 4)) & 15u;
  }
  Vec4f v;
  v.u = ld128(relu_in + off);
  unsigned bits = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) bits |= (v.f[k] > 0 ? 1u : 0u) << k;
  return bits;
}
template <int MASK>
__device__ __forceinline__ bool keep1(const float* relu_in, size_t off) {
  if (MASK == 2) return (reinterpret_cast<const unsigned char*>(relu_in)[off >> 3] >> (off & 7)) & 1u;
  return relu_in[off] > 0;
}

__host__ __device__ inline int bn_slices_for(long long per_channel, int C, int sms) {
  long long s = (static_cast<long long>(sms) * 16 + C - 1) / C;
  const long long max_s = (per_channel + 2047) / 2048;  // >= 2048 elements per slice
  if (s > max_s) s = max_s;
  if (s > kMaxSlices) s = kMaxSlices;
  return static_cast<int>(s < 1 ? 1 : s);
}

template <bool VEC, int MASK>
__global__ void __launch_bounds__(kBlock)
bn_bwd_reduce_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                     const float* __restrict__ relu_in, const float* __restrict__ mean,
                     float2* __restrict__ partial, BnShape sh, int per_slice) {
  __shared__ float sm[32];
  const int c = blockIdx.y, slice = blockIdx.x;
  dependency_wait();
  const float mu = mean[c];
  float s_dy = 0.f, s_dyx = 0.f;
  if (VEC) {
    const int hw4 = sh.HW >> 2, total = sh.N * hw4;
    const int i0 = slice * per_slice, i1 = min(i0 + per_slice, total);
    UnitWalk w(i0 + threadIdx.x, kBlock, hw4);
    for (int i = i0 + threadIdx.x; i < i1; i += kBlock, w.next()) {
      const size_t off = (static_cast<size_t>(w.n) * sh.C + c) * sh.HW + 4 * w.q;
      Vec4f vx, vg, vm;
      vx.u = ld128(x + off);
      vg.u = ld128(dy + off);
      unsigned bits = 15u;
      if (MASK == 1) vm.u = ld128(relu_in + off);
      if (MASK == 2) bits = keep4<2>(relu_in, off);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float g = vg.f[k];
        if (MASK == 1) g = vm.f[k] > 0 ? g : 0.0f;
        if (MASK == 2) g = (bits >> k) & 1u ? g : 0.0f;
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
      if (MASK) g = keep1<MASK>(relu_in, off) ? g : 0.0f;
      s_dy += g;
      s_dyx += g * (x[off] - mu);
    }
  }
  release_dependents();
  s_dy = block_sum(s_dy, sm);
  s_dyx = block_sum(s_dyx, sm);
  if (threadIdx.x == 0)
    partial[static_cast<size_t>(c) * gridDim.x + slice] = make_float2(s_dy, s_dyx);
}

// Units (16-byte vectors, or floats when !VEC) per thread of the apply pass:
// the coefficient lookup and the barrier are paid once per CTA, so more units
// per CTA make them cheaper per byte.
constexpr int kApplyUnits = 4;

template <bool VEC, int MASK>
__global__ void __launch_bounds__(kBlock)
bn_bwd_apply_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                    const float* __restrict__ relu_in, const float* __restrict__ scale,
                    const float* __restrict__ mean, const float* __restrict__ invstd,
                    const float2* __restrict__ partial, int slices, float* __restrict__ dx,
                    float* __restrict__ dscale, float* __restrict__ dbias, BnShape sh) {
  __shared__ float coef[4];
  // channels in DESCENDING order: the reduce pass walked them ascending, so the
  // last ones it touched are the ones most likely still in L2
  const int c = sh.C - 1 - blockIdx.y;
  // issue this thread's loads first, so that their latency overlaps the
  // partial-sum lookup below
  constexpr int kW = VEC ? 4 : 1;
  const int hwu = sh.HW / kW, total = sh.N * hwu;
  const int unit0 = blockIdx.x * (kBlock * kApplyUnits) + threadIdx.x;
  size_t off[kApplyUnits];
  Vec4f vx[kApplyUnits], vg[kApplyUnits], vm[kApplyUnits];
  UnitWalk w(min(unit0, total - 1), kBlock, hwu);
  dependency_wait();
#pragma unroll
  for (int j = 0; j < kApplyUnits; ++j) {
    vx[j].f[0] = vg[j].f[0] = vm[j].f[0] = 0.f;
    off[j] = 0;
    if (unit0 + j * kBlock < total) {
      off[j] = (static_cast<size_t>(w.n) * sh.C + c) * sh.HW + static_cast<size_t>(w.q) * kW;
      if (VEC) {
        vx[j].u = ld128(x + off[j]);
        vg[j].u = ld128(dy + off[j]);
        if (MASK == 1) vm[j].u = ld128(relu_in + off[j]);
        if (MASK == 2) vm[j].i[0] = static_cast<int>(keep4<2>(relu_in, off[j]));
      } else {
        vx[j].f[0] = x[off[j]];
        vg[j].f[0] = dy[off[j]];
        if (MASK == 1) vm[j].f[0] = relu_in[off[j]];
        if (MASK == 2) vm[j].i[0] = keep1<2>(relu_in, off[j]) ? 1 : 0;
      }
      w.next();
    }
  }
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
  release_dependents();
  const float k = coef[0], a = coef[1], b = coef[2], mu = coef[3];
#pragma unroll
  for (int j = 0; j < kApplyUnits; ++j) {
    if (unit0 + j * kBlock >= total) break;
    if (VEC) {
      Vec4f o;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float g = vg[j].f[i];
        if (MASK == 1) g = vm[j].f[i] > 0 ? g : 0.0f;
        if (MASK == 2) g = (vm[j].i[0] >> i) & 1 ? g : 0.0f;
        o.f[i] = k * (g - a - (vx[j].f[i] - mu) * b);
      }
      st128(dx + off[j], o.u);
    } else {
      float g = vg[j].f[0];
      if (MASK == 1) g = vm[j].f[0] > 0 ? g : 0.0f;
      if (MASK == 2) g = vm[j].i[0] & 1 ? g : 0.0f;
      dx[off[j]] = k * (g - a - (vx[j].f[0] - mu) * b);
    }
  }
}

// ----------------------------------------------------------- single pass
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Returns once at most PENDING of this thread's most recent copy groups are still in flight.
template <int PENDING>
__device__ __forceinline__ void cp_async_wait_pending() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}
// A thread issues its copies in kCopyGroups groups, so that it can start adding
// up the units of the first group while the later ones are still in flight
// (a thread only ever reads back what it staged itself: no barrier needed).
constexpr int kCopyGroups = 4;

// CTA size of the single-pass kernel: 512 threads for large shares (fewer
// serial iterations per thread), 256 for small ones.

// Sticky fault word of the cluster kernel's exchange: bit 0 = the wait for the
// peers' pairs ran out of iterations (that launch's outputs are void).
__device__ unsigned g_cluster_faults;

// grid.x = C * CS with cluster dimension CS: the CS CTAs of a cluster share
// channel blockIdx.x / CS.  A "unit" is one float4 (VEC) or one float.
// Dynamic shared memory: 2 * per_cta units (x share, then dy share).
// ADD (only with VEC): the incoming gradient is the join dy + dy_b masked by
// the ReLU input; it is formed while staging, kept in shared memory for the
// two later phases and ALSO written to `joined` for the other consumers of the
// join (the shortcut branch), which replaces a separate join+ReLU kernel.
template <bool VEC, int MASK, int T, bool ADD = false>
__global__ void __launch_bounds__(T)
bn_bwd_cluster_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                      const float* __restrict__ relu_in, const float* __restrict__ scale,
                      const float* __restrict__ mean, const float* __restrict__ invstd,
                      float* __restrict__ dx, float* __restrict__ dscale,
                      float* __restrict__ dbias, BnShape sh, int per_cta,
                      const float* __restrict__ dy_b = nullptr, float* __restrict__ joined = nullptr) {
  extern __shared__ __align__(16) float stage[];
  __shared__ unsigned long long pairs_in;          // mbarrier: counts the peers' pairs as they land
  __shared__ float red[2 * T / 32];
  __shared__ float2 parts[16];   // (sum dy, sum dy*(x-mean)) of every CTA of the cluster
  cg::cluster_group cluster = cg::this_cluster();
  const int cs = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int c = blockIdx.x / cs;
  if (threadIdx.x == 0) {
    mbar_init(&pairs_in, 1);
    fence_mbarrier_init();                            // visible to the peers once the cluster barrier completes
  }
  cluster.barrier_arrive();                           // matched by barrier_wait before the exchange
  constexpr int kW = VEC ? 4 : 1;                     // floats per unit
  const int hwu = sh.HW / kW;                         // units per plane
  const int total = sh.N * hwu;
  const int u0 = min(rank * per_cta, total), u1 = min(u0 + per_cta, total);
  const int first = u0 + threadIdx.x;
  float* sx = stage;
  float* sg = stage + static_cast<size_t>(per_cta) * kW;
  const size_t plane_stride = static_cast<size_t>(sh.C) * sh.HW;
  const size_t chan_off = static_cast<size_t>(c) * sh.HW;
  dependency_wait();                                  // first access to global memory follows
  const float mu = mean[c];
  // units of one copy group per thread (the same in every thread: kCopyGroups * group_units covers a share)
  const int group_units = ((per_cta + T - 1) / T + kCopyGroups - 1) / kCopyGroups;

  // phase 1: stage this CTA's share (asynchronous 16-byte copies, all in flight at once)
  if (VEC && ADD) {
    UnitWalk w(first, T, hwu);
    for (int u = first; u < u1;) {
      // two units per round: x by asynchronous copy, the three gradient-side
      // operands through registers (six independent 16-byte loads in flight)
      Vec4f va[2], vb[2], vr[2];
      size_t offs[2];
      int ls[2], cnt = 0;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (u < u1) {
          offs[j] = w.n * plane_stride + chan_off + static_cast<size_t>(w.q) * 4;
          ls[j] = (u - u0) * 4;
          cp_async16(sx + ls[j], x + offs[j]);
          va[j].u = ld128(dy + offs[j]);
          vb[j].u = ld128(dy_b + offs[j]);
          vr[j].u = ld128(relu_in + offs[j]);
          u += T;
          w.next();
          cnt = j + 1;
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (j < cnt) {
          Vec4f g;
#pragma unroll
          for (int k = 0; k < 4; ++k) g.f[k] = vr[j].f[k] > 0 ? (va[j].f[k] + vb[j].f[k]) : 0.0f;
          *reinterpret_cast<uint4*>(sg + ls[j]) = g.u;
          st128(joined + offs[j], g.u);
        }
      }
    }
  } else if (VEC) {
    UnitWalk w(first, T, hwu);
    int u = first;
#pragma unroll
    for (int g = 0; g < kCopyGroups; ++g) {
      for (int k = 0; k < group_units && u < u1; ++k, u += T, w.next()) {
        const size_t off = w.n * plane_stride + chan_off + static_cast<size_t>(w.q) * 4;
        const int l = (u - u0) * 4;
        cp_async16(sx + l, x + off);
        cp_async16(sg + l, dy + off);
      }
      cp_async_commit();
    }
  } else {
    UnitWalk w(first, T, hwu);
    for (int u = first; u < u1; u += T, w.next()) {
      const size_t off = w.n * plane_stride + chan_off + static_cast<size_t>(w.q);
      const int l = u - u0;
      float g = dy[off];
      if (MASK) g = keep1<MASK>(relu_in, off) ? g : 0.0f;
      sx[l] = x[off];
      sg[l] = g;
    }
  }
  // fused ReLU: while the copies fly, read the ReLU input and keep only the
  // sign decisions, 4 bits per unit (a share is at most 16 units per thread)
  unsigned long long keep = 0;
  if (VEC && MASK == 2 && !ADD) {
    // bit record: one byte holds the decisions of two units
    UnitWalk w(first, T, hwu);
    int slot = 0;
    for (int u = first; u < u1;) {
      // the byte loads of up to 8 units are issued together, then combined
      unsigned char rec[8];
      unsigned shift[8];
      int cnt = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (u < u1) {
          const size_t off = w.n * plane_stride + chan_off + static_cast<size_t>(w.q) * 4;
          rec[j] = reinterpret_cast<const unsigned char*>(relu_in)[off >> 3];
          shift[j] = static_cast<unsigned>(off & 4);
          u += T;
          w.next();
          cnt = j + 1;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < cnt) {
          keep |= static_cast<unsigned long long>((rec[j] >> shift[j]) & 15u) << slot;
          slot += 4;
        }
      }
    }
  } else if (VEC && MASK && !ADD) {
    UnitWalk w(first, T, hwu);
    int slot = 0;
    for (int u = first; u < u1;) {
      // up to 8 independent 16-byte loads in flight per thread, then the sign tests
      Vec4f vm[8];
      int cnt = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (u < u1) {
          const size_t off = w.n * plane_stride + chan_off + static_cast<size_t>(w.q) * 4;
          vm[j].u = ld128(relu_in + off);
          u += T;
          w.next();
          cnt = j + 1;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < cnt) {
          unsigned bits = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) bits |= (vm[j].f[k] > 0 ? 1u : 0u) << k;
          keep |= static_cast<unsigned long long>(bits) << slot;
          slot += 4;
        }
      }
    }
  }
  if (VEC && ADD) cp_async_wait_all();

  // phase 2: partial sums over the share (each thread re-reads what it staged),
  // copy group by copy group as the groups land; the order of the additions is
  // the order of the units, whatever the grouping
  float s_dy = 0.f, s_dyx = 0.f;
  if (VEC) {
    int slot = 0, u = first;
    auto sum_copy_group = [&]() {
      for (int k = 0; k < group_units && u < u1; ++k, u += T, slot += 4) {
        const int l = (u - u0) * 4;
        Vec4f vx, vg;
        vx.u = *reinterpret_cast<const uint4*>(sx + l);
        vg.u = *reinterpret_cast<const uint4*>(sg + l);
        if (MASK && !ADD) {
          const unsigned bits = static_cast<unsigned>(keep >> slot);
#pragma unroll
          for (int q = 0; q < 4; ++q) vg.f[q] = (bits >> q) & 1u ? vg.f[q] : 0.0f;
          *reinterpret_cast<uint4*>(sg + l) = vg.u;    // keep the masked gradient for phase 3
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          s_dy += vg.f[q];
          s_dyx += vg.f[q] * (vx.f[q] - mu);
        }
      }
    };
    static_assert(kCopyGroups == 4, "the waits below are written out for four groups");
    if (!ADD) cp_async_wait_pending<3>();
    sum_copy_group();
    if (!ADD) cp_async_wait_pending<2>();
    sum_copy_group();
    if (!ADD) cp_async_wait_pending<1>();
    sum_copy_group();
    if (!ADD) cp_async_wait_pending<0>();
    sum_copy_group();
  } else {
    for (int u = first; u < u1; u += T) {
      const int l = u - u0;
      s_dy += sg[l];
      s_dyx += sg[l] * (sx[l] - mu);
    }
  }
  // one block reduction for both sums (fixed order), then every CTA pushes its
  // pair into the slot `parts[rank]` of all peers through distributed shared
  // memory; each CTA then owns a full copy, so nobody reads a peer's memory
  // afterwards.
  {
    constexpr int kWarps = T / 32;
    static_assert(kWarps <= 32, "one warp finishes the reduction");
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    s_dy = warp_sum(s_dy);
    s_dyx = warp_sum(s_dyx);
    if (lane == 0) {
      red[wid] = s_dy;
      red[kWarps + wid] = s_dyx;
    }
    __syncthreads();
    if (wid == 0) {
      float p0 = lane < kWarps ? red[lane] : 0.0f;
      float p1 = lane < kWarps ? red[kWarps + lane] : 0.0f;
      p0 = warp_sum(p0);
      p1 = warp_sum(p1);
      cluster.barrier_wait();                       // peers have started: their memory is addressable
      // every pair travels as one asynchronous 8-byte store that also signals the receiver's
      // mbarrier: no second cluster barrier, a CTA goes on as soon as its cs pairs are in
      if (lane == 0) mbar_arrive_expect(&pairs_in, 8u * static_cast<unsigned>(cs));
      if (lane < cs) {
        unsigned remote_slot, remote_bar;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_slot) : "r"(smem_addr(&parts[rank])), "r"(lane));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(smem_addr(&pairs_in)), "r"(lane));
        const unsigned long long bits = (static_cast<unsigned long long>(__float_as_uint(p1)) << 32) |
                                        static_cast<unsigned long long>(__float_as_uint(p0));
        asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b64 [%0], %1, [%2];" ::"r"(remote_slot),
                     "l"(bits), "r"(remote_bar)
                     : "memory");
      }
    } else {
      cluster.barrier_wait();
    }
  }
  // No CTA writes to a peer after this point and none exits before all pairs
  // addressed to it have landed, so the CTAs retire independently.
  {
    bool in = false;
    for (unsigned it = 0; it < (1u << 24) && !in; ++it) in = mbar_try_wait(&pairs_in, 0);
    if (!in) atomicOr(&g_cluster_faults, 1u);
  }

  float a = 0.f, b = 0.f;
  for (int r = 0; r < cs; ++r) {                    // rank order: same totals in every CTA
    a += parts[r].x;
    b += parts[r].y;
  }
  const float r_ = invstd[c];
  const float inv_m = 1.0f / (static_cast<float>(sh.N) * static_cast<float>(sh.HW));
  const float ds = b * r_;
  const float k_ = scale[c] * r_, am = a * inv_m, bm = ds * r_ * inv_m;
  if (rank == 0 && threadIdx.x == 0) {
    dscale[c] = ds;
    dbias[c] = a;
  }

  // phase 3: dx from the staged copy.  From here on this CTA only drains: the
  // next kernel of the stream may take the SM slots that free up.
  release_dependents();
  {
    UnitWalk w(first, T, hwu);
    for (int u = first; u < u1; u += T, w.next()) {
      const size_t off = w.n * plane_stride + chan_off + static_cast<size_t>(w.q) * kW;
      const int l = (u - u0) * kW;
      if (VEC) {
        Vec4f vx, vg, o;
        vx.u = *reinterpret_cast<const uint4*>(sx + l);
        vg.u = *reinterpret_cast<const uint4*>(sg + l);
#pragma unroll
        for (int j = 0; j < 4; ++j) o.f[j] = k_ * (vg.f[j] - am - (vx.f[j] - mu) * bm);
        st128(dx + off, o.u);
      } else {
        dx[off] = k_ * (sg[l] - am - (sx[l] - mu) * bm);
      }
    }
  }
}

// ------------------------------------------- single pass, channel groups
// Planes whose size is not a multiple of four floats (7x7 = 49) cannot be
// moved with 16-byte accesses one channel at a time, but G = 4 / gcd(HW, 4)
// ADJACENT channels of one sample form a contiguous, 16-byte aligned run of
// G*HW floats.  One CTA stages the G channels of all N samples (G*N*HW*8
// bytes of shared memory) with 16-byte copies, reduces every channel with a
// sub-group of its threads from shared memory, overwrites the staged dy with
// dx in place and streams it back with 16-byte stores.
template <int MASK, int G>
__global__ void __launch_bounds__(kBlock)
bn_bwd_group_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                    const float* __restrict__ relu_in, const float* __restrict__ scale,
                    const float* __restrict__ mean, const float* __restrict__ invstd,
                    float* __restrict__ dx, float* __restrict__ dscale,
                    float* __restrict__ dbias, BnShape sh) {
  extern __shared__ __align__(16) float stage[];
  constexpr int kSub = kBlock / G;                    // threads per channel
  __shared__ float red[2][kBlock / 32];
  __shared__ float coef[G][4];
  const int c0 = blockIdx.x * G;
  const int run = G * sh.HW;                          // floats per sample, multiple of 4
  const int run4 = run >> 2;
  const int units = sh.N * run4;
  float* sx = stage;
  float* sg = stage + static_cast<size_t>(sh.N) * run;
  const size_t sample_stride = static_cast<size_t>(sh.C) * sh.HW;
  const size_t base = static_cast<size_t>(c0) * sh.HW;
  UnitWalk wl(threadIdx.x, kBlock, run4);
  dependency_wait();
  if (MASK) {
    // x by asynchronous copy; dy and the ReLU input through registers, four
    // units (eight independent 16-byte loads) per round
    for (int u = threadIdx.x; u < units;) {
      Vec4f vg[4], vm[4];
      unsigned bits[4];
      int us[4], cnt = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (u < units) {
          const size_t off = wl.n * sample_stride + base + 4 * static_cast<size_t>(wl.q);
          cp_async16(sx + 4 * u, x + off);
          vg[j].u = ld128(dy + off);
          if (MASK == 1) vm[j].u = ld128(relu_in + off);
          if (MASK == 2) bits[j] = keep4<2>(relu_in, off);
          us[j] = u;
          u += kBlock;
          wl.next();
          cnt = j + 1;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j < cnt) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (MASK == 1) vg[j].f[k] = vm[j].f[k] > 0 ? vg[j].f[k] : 0.0f;
            if (MASK == 2) vg[j].f[k] = (bits[j] >> k) & 1u ? vg[j].f[k] : 0.0f;
          }
          *reinterpret_cast<uint4*>(sg + 4 * us[j]) = vg[j].u;
        }
      }
    }
  } else {
    for (int u = threadIdx.x; u < units; u += kBlock, wl.next()) {
      const size_t off = wl.n * sample_stride + base + 4 * static_cast<size_t>(wl.q);
      cp_async16(sx + 4 * u, x + off);
      cp_async16(sg + 4 * u, dy + off);
    }
  }
  cp_async_wait_all();
  __syncthreads();
  // channel g is handled by threads [g*kSub, (g+1)*kSub): element (n, i) of the
  // channel sits at staged offset n*run + g*HW + i
  const int g = threadIdx.x / kSub, t = threadIdx.x - g * kSub;
  const int c = c0 + g;
  const float mu = mean[c];
  const int per = sh.N * sh.HW;
  float s_dy = 0.f, s_dyx = 0.f;
  {
    UnitWalk w(t, kSub, sh.HW);                       // (sample, position) without a division per step
    for (int e = t; e < per; e += kSub, w.next()) {
      const int l = w.n * run + g * sh.HW + w.q;
      s_dy += sg[l];
      s_dyx += sg[l] * (sx[l] - mu);
    }
  }
  // reduce inside the sub-group (kSub is a multiple of 32: whole warps per channel)
  s_dy = warp_sum(s_dy);
  s_dyx = warp_sum(s_dyx);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
    red[0][wid] = s_dy;
    red[1][wid] = s_dyx;
  }
  __syncthreads();
  if (t == 0) {
    constexpr int kWarpsPer = kSub / 32;
    float a = 0.f, b = 0.f;
    for (int w = 0; w < kWarpsPer; ++w) {
      a += red[0][g * kWarpsPer + w];
      b += red[1][g * kWarpsPer + w];
    }
    const float r = invstd[c];
    const float inv_m = 1.0f / (static_cast<float>(sh.N) * static_cast<float>(sh.HW));
    const float ds = b * r;
    coef[g][0] = scale[c] * r;
    coef[g][1] = a * inv_m;
    coef[g][2] = ds * r * inv_m;
    coef[g][3] = mu;
    dscale[c] = ds;
    dbias[c] = a;
  }
  __syncthreads();
  const float k_ = coef[g][0], am = coef[g][1], bm = coef[g][2];
  {
    UnitWalk w(t, kSub, sh.HW);
    for (int e = t; e < per; e += kSub, w.next()) {
      const int l = w.n * run + g * sh.HW + w.q;
      sg[l] = k_ * (sg[l] - am - (sx[l] - mu) * bm);        // dx in place
    }
  }
  __syncthreads();
  release_dependents();
  {
    UnitWalk w(threadIdx.x, kBlock, run4);
    for (int u = threadIdx.x; u < units; u += kBlock, w.next()) {
      const size_t off = w.n * sample_stride + base + 4 * static_cast<size_t>(w.q);
      st128(dx + off, *reinterpret_cast<const uint4*>(sg + 4 * u));
    }
  }
}

template <int MASK, int G>
int launch_group(const float* x, const float* dy, const float* relu_in, const float* scale,
                 const float* mean, const float* invstd, float* dx, float* dscale, float* dbias,
                 BnShape sh, cudaStream_t s) {
  auto kernel = bn_bwd_group_kernel<MASK, G>;
  const size_t smem = static_cast<size_t>(G) * sh.N * sh.HW * 8;
  static std::atomic<bool> attr_set[64];
  const int ready = opt_in_once(kernel, attr_set, false);
  if (ready != SGB_OK) return ready;
  return launch_ex(kernel, dim3(sh.C / G), dim3(kBlock), smem, s, 0, true, x, dy, relu_in, scale, mean, invstd,
                   dx, dscale, dbias, sh);
}

// Cluster size (1, 2, 4 or 8) and per-CTA share for the single-pass kernel;
// returns 0 when a channel does not fit 8 CTAs' shared memory.
int cluster_plan(long long units_per_channel, int unit_bytes, int* per_cta, int channels) {
  constexpr int share_kb = 50;   // preferred staging per CTA
  constexpr int max_cs = 8;      // portable cluster size (16-CTA clusters with 50 KB shares measured slower)
  constexpr int fill = 0;        // >0 would split small channels further (measured slower on B200)
  const long long kPreferred = share_kb * 1024LL, kLimit = 100 * 1024;

  for (int pass = 0; pass < 2; ++pass) {
    const long long cap = pass == 0 ? kPreferred : kLimit;
    for (int cs = 1; cs <= max_cs; cs *= 2) {
      long long share = (units_per_channel + cs - 1) / cs;
      if (share * unit_bytes * 2 <= cap && share <= 8192) {   // <= 16 units per thread of a 512-thread CTA
        // Small tensors: a grid of C*cs CTAs that leaves SMs idle is latency
        // bound; split the channel over more CTAs (shorter per-thread loops)
        // while a share still keeps every thread of a 256-thread CTA busy.
        const long long want = static_cast<long long>(sm_count()) * fill;
        while (cs * 2 <= max_cs && static_cast<long long>(channels) * cs < want &&
               (units_per_channel + 2 * cs - 1) / (2 * cs) >= 512) {
          cs *= 2;
          share = (units_per_channel + cs - 1) / cs;
        }
        *per_cta = static_cast<int>(share);
        return cs;
      }
    }
  }
  return 0;
}

template <bool VEC, int MASK, int T, bool ADD = false>
int launch_cluster_t(const float* x, const float* dy, const float* relu_in, const float* scale,
                     const float* mean, const float* invstd, float* dx, float* dscale,
                     float* dbias, BnShape sh, int cs, int per_cta, cudaStream_t s,
                     const float* dy_b = nullptr, float* joined = nullptr) {
  auto kernel = bn_bwd_cluster_kernel<VEC, MASK, T, ADD>;
  const size_t smem = static_cast<size_t>(per_cta) * (VEC ? 16 : 4) * 2;
  static std::atomic<bool> attr_set[64];
  const int ready = opt_in_once(kernel, attr_set, true);
  if (ready != SGB_OK) return ready;
  return launch_ex(kernel, dim3(static_cast<unsigned>(sh.C) * cs), dim3(T), smem, s, cs, true, x, dy, relu_in,
                   scale, mean, invstd, dx, dscale, dbias, sh, per_cta, dy_b, joined);
}

template <bool VEC, int MASK>
int launch_cluster(const float* x, const float* dy, const float* relu_in, const float* scale,
                   const float* mean, const float* invstd, float* dx, float* dscale,
                   float* dbias, BnShape sh, int cs, int per_cta, cudaStream_t s) {
  // at most 16 units per thread (the fused mask keeps 4 bits per unit in 64 bits)
  if (per_cta > 2048)
    return launch_cluster_t<VEC, MASK, 512>(x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias,
                                            sh, cs, per_cta, s);
  return launch_cluster_t<VEC, MASK, 256>(x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias, sh,
                                          cs, per_cta, s);
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

// join + ReLU backward + batch-norm backward.  Uses the single-pass cluster
// kernel when the shape allows it; otherwise the three steps run as separate
// kernels (same values).
int bn_add_relu_backward(const float* x, const float* dy_a, const float* dy_b, const float* relu_in,
                         const float* scale, const float* mean, const float* invstd, float* joined,
                         float* dx, float* dscale, float* dbias, int N, int C, int HW, void* ws,
                         size_t ws_bytes, void* stream);

template <int MASK>
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
  const bool vec = (HW % 4 == 0) && aligned16(x) && aligned16(dy) && aligned16(dx) &&
                   (MASK != 1 || aligned16(relu_in));
  const BnShape sh{N, C, HW};
  if (!vec && HW > 1 && aligned16(x) && aligned16(dy) && aligned16(dx) && (MASK != 1 || aligned16(relu_in))) {
    // odd planes: groups of adjacent channels make 16-byte runs (7x7 layers)
    const int G = (HW % 2) ? 4 : 2;
    if ((HW * G) % 4 == 0 && C % G == 0 && static_cast<long long>(G) * per_channel * 8 <= 100 * 1024) {
      if (G == 4)
        return launch_group<MASK, 4>(x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias, sh, s);
      return launch_group<MASK, 2>(x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias, sh, s);
    }
  }
  {
    int per_cta = 0;
    const int cs = cluster_plan(vec ? per_channel / 4 : per_channel, vec ? 16 : 4, &per_cta, C);
    if (cs > 0 && static_cast<long long>(C) * cs <= 0x7fffffffLL) {
      return vec ? launch_cluster<true, MASK>(x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias,
                                              sh, cs, per_cta, s)
                 : launch_cluster<false, MASK>(x, dy, relu_in, scale, mean, invstd, dx, dscale,
                                               dbias, sh, cs, per_cta, s);
    }
  }
  // channels too large for a cluster: one pass over HBM with the streaming
  // kernel where its plan applies, else two passes
  if (vec && ws && aligned16(ws) && ws_bytes >= bn_stream_workspace_bytes(N, C, HW) &&
      (MASK != 2 || aligned16(relu_in))) {
    BnStreamPlan plan;
    if (bn_stream_plan(N, C, HW, MASK, &plan))
      return bn_stream_backward(MASK, x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias, N, C, HW, plan, ws, s);
  }
  const int slices = bn_slices_for(per_channel, C, sm_count());
  if (!ws || ws_bytes < static_cast<size_t>(slices) * C * sizeof(float2) || !aligned16(ws))
    return SGB_ERR_WORKSPACE;
  float2* partial = static_cast<float2*>(ws);
  const int total = static_cast<int>(vec ? per_channel / 4 : per_channel);
  const int per_slice = static_cast<int>(ceil_div(total, slices));
  const dim3 g1(slices, C), g2(static_cast<unsigned>(ceil_div(total, kBlock * kApplyUnits)), C);
  int st;
  if (vec) {
    st = launch_ex(bn_bwd_reduce_kernel<true, MASK>, g1, dim3(kBlock), 0, s, 0, true, x, dy, relu_in, mean, partial,
                   sh, per_slice);
    if (st != SGB_OK) return st;
    st = launch_ex(bn_bwd_apply_kernel<true, MASK>, g2, dim3(kBlock), 0, s, 0, true, x, dy, relu_in, scale, mean,
                   invstd, partial, slices, dx, dscale, dbias, sh);
  } else {
    st = launch_ex(bn_bwd_reduce_kernel<false, MASK>, g1, dim3(kBlock), 0, s, 0, true, x, dy, relu_in, mean,
                   partial, sh, per_slice);
    if (st != SGB_OK) return st;
    st = launch_ex(bn_bwd_apply_kernel<false, MASK>, g2, dim3(kBlock), 0, s, 0, true, x, dy, relu_in, scale, mean,
                   invstd, partial, slices, dx, dscale, dbias, sh);
  }
  return st;
}

int bn_add_relu_backward(const float* x, const float* dy_a, const float* dy_b, const float* relu_in,
                         const float* scale, const float* mean, const float* invstd, float* joined,
                         float* dx, float* dscale, float* dbias, int N, int C, int HW, void* ws,
                         size_t ws_bytes, void* stream) {
  if (N < 0 || C < 0 || HW < 0) return SGB_ERR_SIZE;
  if (N == 0 || C == 0 || HW == 0) return SGB_OK;
  if (!x || !dy_a || !dy_b || !relu_in || !scale || !mean || !invstd || !joined || !dx || !dscale ||
      !dbias)
    return SGB_ERR_NULL;
  const long long per_channel = static_cast<long long>(N) * HW;
  if (per_channel > 0x7fffffffLL || C > 65535) return SGB_ERR_SIZE;
  const bool vec = (HW % 4 == 0) && aligned16(x) && aligned16(dy_a) && aligned16(dy_b) &&
                   aligned16(relu_in) && aligned16(joined) && aligned16(dx);
  if (vec) {
    int per_cta = 0;
    const int cs = cluster_plan(per_channel / 4, 16, &per_cta, C);
    if (cs > 0 && static_cast<long long>(C) * cs <= 0x7fffffffLL) {
      const BnShape sh{N, C, HW};
      cudaStream_t s = as_stream(stream);
      if (per_cta > 2048)
        return launch_cluster_t<true, true, 512, true>(x, dy_a, relu_in, scale, mean, invstd, dx, dscale,
                                                       dbias, sh, cs, per_cta, s, dy_b, joined);
      return launch_cluster_t<true, true, 256, true>(x, dy_a, relu_in, scale, mean, invstd, dx, dscale,
                                                     dbias, sh, cs, per_cta, s, dy_b, joined);
    }
  }
  int st = sgb_add_relu_backward_f32(dy_a, dy_b, relu_in, joined, static_cast<size_t>(N) * C * HW, stream);
  if (st != SGB_OK) return st;
  return bn_backward<0>(x, joined, nullptr, scale, mean, invstd, dx, dscale, dbias, N, C, HW, ws,
                        ws_bytes, stream);
}

// ------------------------------------------------------------ forward (training)
// Forward partner of the backward kernels: batch statistics, normalisation and
// running-statistics update in one pass over x.  A cluster stages its channel
// in shared memory once; mean and the centred sum of squares are two reductions
// over the staged copy (no E[x^2]-E[x]^2 cancellation), each exchanged through
// distributed shared memory.  Emits what the backward consumes: save_mean and
// save_invstd = 1/sqrt(biased_var + eps).  Running statistics follow cuDNN:
// r = (1-f)*r + f*batch_value, with the UNBIASED variance (M/(M-1)).
template <bool VEC, int T>
__global__ void __launch_bounds__(T)
bn_fwd_cluster_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                      const float* __restrict__ bias, float* __restrict__ running_mean,
                      float* __restrict__ running_var, float factor, float eps,
                      float* __restrict__ y, float* __restrict__ save_mean,
                      float* __restrict__ save_invstd, BnShape sh, int per_cta) {
  extern __shared__ __align__(16) float stage[];
  __shared__ float red[T / 32];
  __shared__ float parts[2][16];
  cg::cluster_group cluster = cg::this_cluster();
  const int cs = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int c = blockIdx.x / cs;
  cluster.barrier_arrive();
  constexpr int kW = VEC ? 4 : 1;
  const int hwu = sh.HW / kW, total = sh.N * hwu;
  const int u0 = min(rank * per_cta, total), u1 = min(u0 + per_cta, total);
  const int first = u0 + threadIdx.x;
  const size_t plane_stride = static_cast<size_t>(sh.C) * sh.HW;
  const size_t chan_off = static_cast<size_t>(c) * sh.HW;
  {
    UnitWalk w(first, T, hwu);
    for (int u = first; u < u1; u += T, w.next()) {
      const size_t off = w.n * plane_stride + chan_off + static_cast<size_t>(w.q) * kW;
      if (VEC) cp_async16(stage + (u - u0) * 4, x + off);
      else stage[u - u0] = x[off];
    }
  }
  if (VEC) cp_async_wait_all();
  const float inv_m = 1.0f / (static_cast<float>(sh.N) * static_cast<float>(sh.HW));
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  constexpr int kWarps = T / 32;
  auto cluster_total = [&](float v, int slot) -> float {
    v = warp_sum(v);
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
      float p = lane < kWarps ? red[lane] : 0.0f;
      p = warp_sum(p);
      if (slot == 0) cluster.barrier_wait();      // first exchange: peers must have started
      if (lane < cs) *cluster.map_shared_rank(&parts[slot][rank], lane) = p;
    } else if (slot == 0) {
      cluster.barrier_wait();
    }
    cluster.sync();
    float t = 0.f;
    for (int r = 0; r < cs; ++r) t += parts[slot][r];
    return t;
  };
  float s = 0.f;
  for (int u = first; u < u1; u += T) {
    const int l = (u - u0) * kW;
#pragma unroll
    for (int k = 0; k < kW; ++k) s += stage[l + k];
  }
  const float mu = cluster_total(s, 0) * inv_m;
  float q = 0.f;
  for (int u = first; u < u1; u += T) {
    const int l = (u - u0) * kW;
#pragma unroll
    for (int k = 0; k < kW; ++k) {
      const float d = stage[l + k] - mu;
      q += d * d;
    }
  }
  const float var = cluster_total(q, 1) * inv_m;      // biased
  const float invstd = 1.0f / sqrtf(var + eps);
  if (rank == 0 && threadIdx.x == 0) {
    save_mean[c] = mu;
    save_invstd[c] = invstd;
    const float m = static_cast<float>(sh.N) * static_cast<float>(sh.HW);
    const float unbiased = m > 1.0f ? var * (m / (m - 1.0f)) : var;
    running_mean[c] = (1.0f - factor) * running_mean[c] + factor * mu;
    running_var[c] = (1.0f - factor) * running_var[c] + factor * unbiased;
  }
  const float g = scale[c] * invstd, b = bias[c];
  {
    UnitWalk w(first, T, hwu);
    for (int u = first; u < u1; u += T, w.next()) {
      const size_t off = w.n * plane_stride + chan_off + static_cast<size_t>(w.q) * kW;
      const int l = (u - u0) * kW;
      if (VEC) {
        Vec4f v, o;
        v.u = *reinterpret_cast<const uint4*>(stage + l);
#pragma unroll
        for (int k = 0; k < 4; ++k) o.f[k] = (v.f[k] - mu) * g + b;
        st128(y + off, o.u);
      } else {
        y[off] = (stage[l] - mu) * g + b;
      }
    }
  }
}

// Fallback for channels that do not fit a cluster: three streaming kernels
// (mean partials, centred-square partials, normalise), partials in workspace.
template <int PHASE>
__global__ void __launch_bounds__(kBlock)
bn_fwd_partial_kernel(const float* __restrict__ x, const float* __restrict__ mean_in,
                      float* __restrict__ partial, BnShape sh, int per_slice) {
  __shared__ float sm[32];
  const int c = blockIdx.y, slice = blockIdx.x;
  const int total = sh.N * sh.HW;
  const int i0 = slice * per_slice, i1 = min(i0 + per_slice, total);
  const float mu = PHASE == 1 ? mean_in[c] : 0.0f;
  float acc = 0.f;
  UnitWalk w(i0 + threadIdx.x, kBlock, sh.HW);
  for (int i = i0 + threadIdx.x; i < i1; i += kBlock, w.next()) {
    const float v = x[(static_cast<size_t>(w.n) * sh.C + c) * sh.HW + w.q];
    acc += PHASE == 0 ? v : (v - mu) * (v - mu);
  }
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) partial[static_cast<size_t>(c) * gridDim.x + slice] = acc;
}

__global__ void bn_fwd_finish_kernel(int phase, const float* __restrict__ partial, int slices,
                                     float* __restrict__ save_mean, float* __restrict__ save_invstd,
                                     float* __restrict__ running_mean, float* __restrict__ running_var,
                                     float factor, float eps, BnShape sh) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= sh.C) return;
  float t = 0.f;
  for (int k = 0; k < slices; ++k) t += partial[static_cast<size_t>(c) * slices + k];
  const float m = static_cast<float>(sh.N) * static_cast<float>(sh.HW);
  if (phase == 0) {
    save_mean[c] = t / m;
  } else {
    const float var = t / m;
    save_invstd[c] = 1.0f / sqrtf(var + eps);
    const float unbiased = m > 1.0f ? var * (m / (m - 1.0f)) : var;
    running_mean[c] = (1.0f - factor) * running_mean[c] + factor * save_mean[c];
    running_var[c] = (1.0f - factor) * running_var[c] + factor * unbiased;
  }
}

__global__ void __launch_bounds__(kBlock)
bn_fwd_normalize_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                        const float* __restrict__ bias, const float* __restrict__ mean,
                        const float* __restrict__ invstd, float* __restrict__ y, BnShape sh) {
  const int c = blockIdx.y;
  const int i = blockIdx.x * kBlock + threadIdx.x;
  if (i >= sh.N * sh.HW) return;
  const int n = i / sh.HW, q = i - n * sh.HW;
  const size_t off = (static_cast<size_t>(n) * sh.C + c) * sh.HW + q;
  y[off] = (x[off] - mean[c]) * (scale[c] * invstd[c]) + bias[c];
}

template <bool VEC, int T>
int launch_fwd_cluster(const float* x, const float* scale, const float* bias, float* rm, float* rv,
                       float factor, float eps, float* y, float* sm_, float* si, BnShape sh, int cs,
                       int per_cta, cudaStream_t s) {
  auto kernel = bn_fwd_cluster_kernel<VEC, T>;
  const size_t smem = static_cast<size_t>(per_cta) * (VEC ? 16 : 4);
  static std::atomic<bool> attr_set[64];
  const int ready = opt_in_once(kernel, attr_set, false);
  if (ready != SGB_OK) return ready;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sh.C) * cs);
  cfg.blockDim = dim3(T);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, x, scale, bias, rm, rv, factor, eps, y, sm_, si, sh, per_cta);
  if (e != cudaSuccess) return note_cuda_error(e);
  return launch_status();
}

int bn_forward_training(const float* x, const float* scale, const float* bias, float* rm, float* rv,
                        float factor, float eps, float* y, float* save_mean, float* save_invstd,
                        int N, int C, int HW, void* ws, size_t ws_bytes, void* stream) {
  if (N < 0 || C < 0 || HW < 0) return SGB_ERR_SIZE;
  if (N == 0 || C == 0 || HW == 0) return SGB_OK;
  if (!x || !scale || !bias || !rm || !rv || !y || !save_mean || !save_invstd) return SGB_ERR_NULL;
  const long long per_channel = static_cast<long long>(N) * HW;
  if (per_channel > 0x7fffffffLL || C > 65535) return SGB_ERR_SIZE;
  cudaStream_t s = as_stream(stream);
  const BnShape sh{N, C, HW};
  const bool vec = (HW % 4 == 0) && aligned16(x) && aligned16(y);
  // x only is staged: a share of `units` units costs units * unit_bytes
  const long long units = vec ? per_channel / 4 : per_channel;
  const int unit_bytes = vec ? 16 : 4;
  for (int pass = 0; pass < 2; ++pass) {
    const long long cap = pass == 0 ? 50 * 1024 : 100 * 1024;
    for (int cs = 1; cs <= 8; cs *= 2) {
      const long long share = (units + cs - 1) / cs;
      if (share * unit_bytes <= cap) {
        const int per_cta = static_cast<int>(share);
        if (vec)
          return share > 2048
                     ? launch_fwd_cluster<true, 512>(x, scale, bias, rm, rv, factor, eps, y, save_mean, save_invstd, sh, cs, per_cta, s)
                     : launch_fwd_cluster<true, 256>(x, scale, bias, rm, rv, factor, eps, y, save_mean, save_invstd, sh, cs, per_cta, s);
        return launch_fwd_cluster<false, 256>(x, scale, bias, rm, rv, factor, eps, y, save_mean, save_invstd, sh, cs, per_cta, s);
      }
    }
  }
  const int slices = bn_slices_for(per_channel, C, sm_count());
  if (!ws || ws_bytes < static_cast<size_t>(slices) * C * sizeof(float)) return SGB_ERR_WORKSPACE;
  float* partial = static_cast<float*>(ws);
  const int per_slice = static_cast<int>(ceil_div(static_cast<size_t>(per_channel), slices));
  const dim3 g1(slices, C);
  const unsigned fb = static_cast<unsigned>(ceil_div(C, 128));
  bn_fwd_partial_kernel<0><<<g1, kBlock, 0, s>>>(x, nullptr, partial, sh, per_slice);
  bn_fwd_finish_kernel<<<fb, 128, 0, s>>>(0, partial, slices, save_mean, save_invstd, rm, rv, factor, eps, sh);
  bn_fwd_partial_kernel<1><<<g1, kBlock, 0, s>>>(x, save_mean, partial, sh, per_slice);
  bn_fwd_finish_kernel<<<fb, 128, 0, s>>>(1, partial, slices, save_mean, save_invstd, rm, rv, factor, eps, sh);
  bn_fwd_normalize_kernel<<<dim3(static_cast<unsigned>(ceil_div(static_cast<size_t>(per_channel), kBlock)), C),
                            kBlock, 0, s>>>(x, scale, bias, save_mean, save_invstd, y, sh);
  return launch_status();
}

// ------------------------------------------------ variant with built-in scratch
// Partial sums of the two-pass scheme for callers that cannot provide a
// workspace: a fixed array that lives in the library's device image.  Every
// GPU that loads the library holds these 2 MiB until the process exits.
constexpr int kNoAllocMaxChannels = 4096;
static __device__ __align__(256) float2 g_bn_static_scratch[kMaxSlices * kNoAllocMaxChannels];

// In host code `g_bn_static_scratch` is only a handle for the symbol, not an
// address a kernel could use; the device address is looked up once per device
// (with that device current) and cached here.
float2* static_scratch_address(int* status) {
  static std::atomic<float2*> cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    *status = note_cuda_error(e);
    return nullptr;
  }
  if (dev < 0 || dev >= 64) {
    *status = SGB_ERR_UNSUPPORTED;
    return nullptr;
  }
  if (!cached[dev].load(std::memory_order_acquire)) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_bn_static_scratch);
    if (e != cudaSuccess || !ptr) {
      *status = note_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
      return nullptr;
    }
    cached[dev].store(static_cast<float2*>(ptr), std::memory_order_release);
  }
  *status = SGB_OK;
  return cached[dev].load(std::memory_order_acquire);
}

int bn_backward_static(const float* x, const float* dy, const float* scale, const float* mean,
                       const float* invstd, float* dx, float* dscale, float* dbias, int N, int C,
                       int HW, void* stream) {
  if (N < 0 || C < 0 || HW < 0) return SGB_ERR_SIZE;
  if (N == 0 || C == 0 || HW == 0) return SGB_OK;
  if (!x || !dy || !scale || !mean || !invstd || !dx || !dscale || !dbias) return SGB_ERR_NULL;
  if (C > kNoAllocMaxChannels) return SGB_ERR_LIMIT;   // the built-in scratch holds 4096 channels
  const long long per_channel = static_cast<long long>(N) * HW;
  if (per_channel > 0x7fffffffLL) return SGB_ERR_SIZE;
  int st = SGB_OK;
  float2* partial = static_scratch_address(&st);
  if (!partial) return st;
  cudaStream_t s = as_stream(stream);
  const int slices = bn_slices_for(per_channel, C, sm_count());   // <= kMaxSlices
  const bool vec = (HW % 4 == 0) && aligned16(x) && aligned16(dy) && aligned16(dx);
  const BnShape sh{N, C, HW};
  const int total = static_cast<int>(vec ? per_channel / 4 : per_channel);
  const int per_slice = static_cast<int>(ceil_div(total, slices));
  const dim3 g1(slices, C), g2(static_cast<unsigned>(ceil_div(total, kBlock * kApplyUnits)), C);
  // pass 1 writes partial[c * slices + k] for every k < slices before pass 2
  // (same stream) reads exactly those entries, so nothing has to be cleared
  if (vec) {
    bn_bwd_reduce_kernel<true, false><<<g1, kBlock, 0, s>>>(x, dy, nullptr, mean, partial, sh, per_slice);
    bn_bwd_apply_kernel<true, false><<<g2, kBlock, 0, s>>>(x, dy, nullptr, scale, mean, invstd, partial,
                                                           slices, dx, dscale, dbias, sh);
  } else {
    bn_bwd_reduce_kernel<false, false><<<g1, kBlock, 0, s>>>(x, dy, nullptr, mean, partial, sh, per_slice);
    bn_bwd_apply_kernel<false, false><<<g2, kBlock, 0, s>>>(x, dy, nullptr, scale, mean, invstd, partial,
                                                            slices, dx, dscale, dbias, sh);
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

int sgb_bn_backward_faults(unsigned* flags) {
  if (!flags) return SGB_ERR_NULL;
  unsigned streaming = 0, cluster = 0;
  const int st = bn_stream_faults(&streaming);
  if (st != SGB_OK) return st;
  cudaError_t e = cudaMemcpyFromSymbol(&cluster, g_cluster_faults, sizeof(unsigned));
  if (e != cudaSuccess) return note_cuda_error(e);
  *flags = streaming | (cluster << 8);
  return SGB_OK;
}

int sgb_bn_backward_stream_plan(int N, int C, int HW, int mask, int* plan6) {
  if (!plan6) return SGB_ERR_NULL;
  BnStreamPlan p;
  if (!bn_stream_plan(N, C, HW, mask, &p)) return 0;
  plan6[0] = p.P;
  plan6[1] = p.Lp;
  plan6[2] = p.S;
  plan6[3] = p.parts;
  plan6[4] = p.depth;
  plan6[5] = p.arrays;
  return 1;
}

int sgb_bn_backward_f32(const float* x, const float* dy, const float* scale, const float* mean,
                        const float* invstd, float* dx, float* dscale, float* dbias, int N,
                        int C, int HW, void* ws, size_t ws_bytes, void* stream) {
  return bn_backward<0>(x, dy, nullptr, scale, mean, invstd, dx, dscale, dbias, N, C, HW,
                        ws, ws_bytes, stream);
}

int sgb_bn_add_relu_backward_f32(const float* x, const float* dy_a, const float* dy_b,
                                 const float* relu_in, const float* scale, const float* mean,
                                 const float* invstd, float* joined, float* dx, float* dscale,
                                 float* dbias, int N, int C, int HW, void* ws, size_t ws_bytes,
                                 void* stream) {
  return bn_add_relu_backward(x, dy_a, dy_b, relu_in, scale, mean, invstd, joined, dx, dscale, dbias, N,
                              C, HW, ws, ws_bytes, stream);
}

int sgb_bn_forward_training_f32(const float* x, const float* scale, const float* bias,
                                float* running_mean, float* running_var, float factor, float eps,
                                float* y, float* save_mean, float* save_invstd, int N, int C,
                                int HW, void* ws, size_t ws_bytes, void* stream) {
  return bn_forward_training(x, scale, bias, running_mean, running_var, factor, eps, y, save_mean,
                             save_invstd, N, C, HW, ws, ws_bytes, stream);
}

int sgb_bn_backward_noalloc_f32(const float* x, const float* dy, const float* scale,
                                const float* mean, const float* invstd, float* dx, float* dscale,
                                float* dbias, int N, int C, int HW, void* stream) {
  return bn_backward_static(x, dy, scale, mean, invstd, dx, dscale, dbias, N, C, HW, stream);
}

int sgb_bn_relu_backward_mask_f32(const float* x, const float* dy, const void* relu_mask,
                                  const float* scale, const float* mean, const float* invstd,
                                  float* dx, float* dscale, float* dbias, int N, int C, int HW,
                                  void* ws, size_t ws_bytes, void* stream) {
  return bn_backward<2>(x, dy, static_cast<const float*>(relu_mask), scale, mean, invstd, dx, dscale, dbias, N, C,
                        HW, ws, ws_bytes, stream);
}

int sgb_bn_relu_backward_f32(const float* x, const float* dy, const float* relu_in,
                             const float* scale, const float* mean, const float* invstd,
                             float* dx, float* dscale, float* dbias, int N, int C, int HW,
                             void* ws, size_t ws_bytes, void* stream) {
  return bn_backward<1>(x, dy, relu_in, scale, mean, invstd, dx, dscale, dbias, N, C, HW,
                        ws, ws_bytes, stream);
}

}  // extern "C"
