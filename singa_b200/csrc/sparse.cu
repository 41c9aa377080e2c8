// Gradient sparsification kernels of the communicator:
//   * threshold selection with residual correction and ORDER-PRESERVING
//     compaction into a [1-based index | value] payload;
//   * top-K selection by radix select on a 32-bit key (no sort), ties broken
//     by lower index, with the same compaction;
//   * scatter-add of a received payload into the dense sum buffer.
//
// Compaction is the classic three-step form (per-tile counts, one-CTA scan of
// the tile counts, per-tile write at the scanned offsets).  It has no waits
// between CTAs, so nothing can spin.  All index arithmetic that reaches the
// payload is 1-based int32, the reference's wire format.
#include "common.cuh"

namespace sgb {
namespace {

constexpr int kBlock = 256;
constexpr int kVecPerThread = 4;                       // float4 vectors per thread
constexpr int kTile = kBlock * kVecPerThread * 4;      // 4096 elements per CTA
constexpr int kBins1 = 4096, kBins23 = 1024;           // 12 + 10 + 10 key bits

// Device-resident selection state shared by the top-K passes.
struct SelectState {
  unsigned prefix;       // key bits decided so far (high bits), low bits zero
  unsigned remaining;    // how many elements are still to be taken at/below prefix
  unsigned threshold;    // final key T
  unsigned quota;        // number of key == T elements to take (lowest indices)
  int nnz;               // payload length (threshold mode: count; top-K: K)
  unsigned max_key;      // largest key seen by pass 0 (zeroed with the histogram before every call)
  unsigned skip1;        // 1: every key is below 2^10, pass 1 (bits 10..19) has nothing to decide
  int pad;
};

// Workspace layout (all 256-byte aligned segments).
struct Workspace {
  unsigned* tile_counts;   // tiles entries (threshold) or packed gt<<16|eq... see below
  unsigned* tile_gt;       // tiles
  unsigned* tile_eq;       // tiles
  unsigned* hist;          // kBins1
  SelectState* state;
};
inline size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
inline size_t tiles_of(size_t n) { return ceil_div(n, kTile); }
inline size_t workspace_bytes(size_t n) {
  return 3 * align256(tiles_of(n) * sizeof(unsigned)) + align256(kBins1 * sizeof(unsigned)) +
         align256(sizeof(SelectState));
}
inline Workspace carve(void* ws, size_t n) {
  char* p = static_cast<char*>(ws);
  Workspace w;
  const size_t t = align256(tiles_of(n) * sizeof(unsigned));
  w.tile_counts = reinterpret_cast<unsigned*>(p); p += t;
  w.tile_gt = reinterpret_cast<unsigned*>(p); p += t;
  w.tile_eq = reinterpret_cast<unsigned*>(p); p += t;
  w.hist = reinterpret_cast<unsigned*>(p); p += align256(kBins1 * sizeof(unsigned));
  w.state = reinterpret_cast<SelectState*>(p);
  return w;
}

// ------------------------------------------------------------- tile helpers
// Element order inside a tile: vector v = r * kBlock + t (round r, thread t),
// elements 4v .. 4v+3.  Loads are fully coalesced; ranks below follow this
// order, which is ascending element index.
__device__ __forceinline__ float load_sum(const float* __restrict__ g,
                                          const float* __restrict__ acc, size_t i) {
  return acc ? g[i] + acc[i] : g[i];
}

// The four values s = g (+ acc) of elements i .. i+3; out-of-range lanes get 0.
// `vec` (host-checked 16-byte alignment of g and acc) turns the eight scalar
// loads into two 128-bit loads.
__device__ __forceinline__ void load_sum4(const float* __restrict__ g,
                                          const float* __restrict__ acc, size_t i, size_t n,
                                          bool vec, float (&s)[4]) {
  if (vec && i + 4 <= n) {
    const float4 a = *reinterpret_cast<const float4*>(g + i);
    s[0] = a.x; s[1] = a.y; s[2] = a.z; s[3] = a.w;
    if (acc) {
      const float4 b = *reinterpret_cast<const float4*>(acc + i);
      s[0] += b.x; s[1] += b.y; s[2] += b.z; s[3] += b.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j] = i + j < n ? load_sum(g, acc, i + j) : 0.0f;
  }
}

__device__ __forceinline__ void store4(float* __restrict__ p, size_t i, size_t n, bool vec,
                                       const float (&v)[4]) {
  if (vec && i + 4 <= n) {
    *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i + j < n) p[i + j] = v[j];
  }
}

// Exclusive offsets, in element order, of per-thread per-round counts c[r].
// Returns the tile total.  smem: 32 unsigned.
__device__ __forceinline__ unsigned tile_exclusive(const unsigned (&c)[kVecPerThread],
                                                   unsigned (&excl)[kVecPerThread],
                                                   unsigned* smem) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;  // 8 warps
  unsigned incl[kVecPerThread];
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    unsigned v = c[r];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    incl[r] = v;
    if (lane == 31) smem[r * 8 + w] = v;  // warp total for (round r, warp w)
  }
  __syncthreads();
  if (w == 0) {  // scan the 32 (round, warp) totals in element order
    unsigned v = smem[lane];
    unsigned s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned u = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += u;
    }
    smem[lane] = s - v;          // exclusive
    if (lane == 31) smem[32] = s;  // tile total
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) excl[r] = smem[r * 8 + w] + incl[r] - c[r];
  const unsigned total = smem[32];
  __syncthreads();
  return total;
}

// ------------------------------------------------------------ threshold mode
// kept value of element i: s = g (+ acc); |s| >= thr ? s : 0; sent iff != 0.
// With a residual buffer the count pass leaves s = g + acc IN acc, so that the
// write pass reads 4 bytes per element instead of 8 and only has to zero the
// entries it sends (the residual of every other element is s itself).
__global__ void __launch_bounds__(kBlock)
thr_count_kernel(const float* __restrict__ g, float* __restrict__ acc, size_t n,
                 float thr, unsigned* __restrict__ tile_counts, bool vec) {
  __shared__ unsigned sm[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * kTile;
  unsigned cnt = 0;
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    float s[4];
    load_sum4(g, acc, i, n, vec, s);      // out-of-range lanes are 0 and never counted
    if (acc) store4(acc, i, n, vec, s);
#pragma unroll
    for (int j = 0; j < 4; ++j) cnt += (fabsf(s[j]) >= thr && s[j] != 0.0f) ? 1u : 0u;
  }
  // block total (integer, order irrelevant)
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned t = 0;
    for (int k = 0; k < kBlock / 32; ++k) t += sm[k];
    tile_counts[blockIdx.x] = t;
  }
}

// One CTA: exclusive scan of the tile counts (two arrays at once), totals to
// the state.  In place: counts become offsets.  Every thread owns a contiguous
// chunk: it adds the chunk up, a block-wide scan of the 1024 chunk totals gives
// its base, and a second walk over the chunk writes the offsets.
__global__ void __launch_bounds__(1024)
scan_tiles_kernel(unsigned* __restrict__ a, unsigned* __restrict__ b, size_t tiles,
                  SelectState* __restrict__ st, int write_nnz) {
  __shared__ unsigned sa[32], sb[32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const size_t chunk = (tiles + 1023) / 1024;
  const size_t lo = threadIdx.x * chunk, hi = lo + chunk < tiles ? lo + chunk : tiles;
  constexpr int kReg = 32;                 // chunks up to 32 entries live in registers
  const bool in_regs = chunk <= kReg;
  unsigned ra_[kReg], rb_[kReg];
  unsigned ta = 0, tb = 0;
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < kReg; ++j) {       // independent loads, one round trip
      const size_t i = lo + j;
      ra_[j] = (j < static_cast<int>(chunk) && i < tiles) ? a[i] : 0u;
      rb_[j] = (b && j < static_cast<int>(chunk) && i < tiles) ? b[i] : 0u;
    }
#pragma unroll
    for (int j = 0; j < kReg; ++j) {
      ta += ra_[j];
      tb += rb_[j];
    }
  } else {
    for (size_t i = lo; i < hi; ++i) {
      ta += a[i];
      if (b) tb += b[i];
    }
  }
  unsigned xa = ta, xb = tb;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned ua = __shfl_up_sync(0xffffffffu, xa, o);
    const unsigned ub = __shfl_up_sync(0xffffffffu, xb, o);
    if (lane >= o) { xa += ua; xb += ub; }
  }
  if (lane == 31) { sa[w] = xa; sb[w] = xb; }
  __syncthreads();
  if (w == 0) {
    const unsigned va = sa[lane], vb = sb[lane];
    unsigned ya = va, yb = vb;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned ua = __shfl_up_sync(0xffffffffu, ya, o);
      const unsigned ub = __shfl_up_sync(0xffffffffu, yb, o);
      if (lane >= o) { ya += ua; yb += ub; }
    }
    sa[lane] = ya - va;
    sb[lane] = yb - vb;
    if (lane == 31 && write_nnz) st->nnz = static_cast<int>(ya);
  }
  __syncthreads();
  unsigned ra = sa[w] + xa - ta, rb = sb[w] + xb - tb;   // exclusive base of this chunk
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < kReg; ++j) {
      const size_t i = lo + j;
      if (j < static_cast<int>(chunk) && i < tiles) {
        a[i] = ra;
        ra += ra_[j];
        if (b) {
          b[i] = rb;
          rb += rb_[j];
        }
      }
    }
    return;
  }
  for (size_t i = lo; i < hi; ++i) {
    const unsigned va = a[i];
    a[i] = ra;
    ra += va;
    if (b) {
      const unsigned vb = b[i];
      b[i] = rb;
      rb += vb;
    }
  }
}

// `sum` is acc after the count pass (or g when there is no residual buffer).
__global__ void __launch_bounds__(kBlock)
thr_write_kernel(const float* __restrict__ sum, float* __restrict__ acc, size_t n, float thr,
                 const unsigned* __restrict__ tile_offsets, int* __restrict__ idx_out,
                 float* __restrict__ val_out, const SelectState* __restrict__ st, bool vec) {
  __shared__ unsigned sm[33];
  // packed payload [idx(nnz) | val(nnz)]: values start right after the indices
  if (!val_out) val_out = reinterpret_cast<float*>(idx_out) + st->nnz;
  const size_t base = static_cast<size_t>(blockIdx.x) * kTile;
  float kept[kVecPerThread][4];
  unsigned c[kVecPerThread], excl[kVecPerThread];
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    c[r] = 0;
    float s[4], res[4];
    load_sum4(sum, nullptr, i, n, vec, s);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float k = fabsf(s[j]) >= thr ? s[j] : 0.0f;   // out-of-range lanes: s == 0 -> k == 0
      res[j] = s[j] - k;                                  // residual kept locally
      kept[r][j] = k;
      c[r] += k != 0.0f ? 1u : 0u;
    }
    if (acc && c[r]) store4(acc, i, n, vec, res);         // untouched vectors already hold their residual
  }
  tile_exclusive(c, excl, sm);
  const unsigned tile_off = tile_offsets[blockIdx.x];
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    unsigned pos = tile_off + excl[r];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (kept[r][j] != 0.0f) {
        idx_out[pos] = static_cast<int>(i + j + 1);
        val_out[pos] = kept[r][j];
        ++pos;
      }
  }
}

// Capacity-bounded form: the payload layout is fixed, [idx(cap) | val(cap)],
// and only the first `cap` selected entries (index order) are written.  The
// others stay in the residual (acc keeps s there), so they are sent by a later
// call; their number is added to *dropped.  With this the length of the
// exchange is known on the host before the count is, and the caller needs no
// host round trip between selection and all-gather.
__global__ void __launch_bounds__(kBlock)
thr_write_bounded_kernel(const float* __restrict__ sum, float* __restrict__ acc, size_t n, float thr,
                         const unsigned* __restrict__ tile_offsets, int* __restrict__ idx_out, unsigned cap,
                         unsigned long long* __restrict__ dropped, bool vec) {
  __shared__ unsigned sm[33];
  float* val_out = reinterpret_cast<float*>(idx_out) + cap;
  const size_t base = static_cast<size_t>(blockIdx.x) * kTile;
  float sv[kVecPerThread][4];
  unsigned c[kVecPerThread], excl[kVecPerThread];
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    c[r] = 0;
    load_sum4(sum, nullptr, i, n, vec, sv[r]);
#pragma unroll
    for (int j = 0; j < 4; ++j) c[r] += (fabsf(sv[r][j]) >= thr && sv[r][j] != 0.0f) ? 1u : 0u;
  }
  tile_exclusive(c, excl, sm);
  const unsigned tile_off = tile_offsets[blockIdx.x];
  unsigned lost = 0;
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    if (!c[r]) continue;                                  // untouched vectors already hold their residual
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    unsigned pos = tile_off + excl[r];
    bool sent = false;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (fabsf(sv[r][j]) >= thr && sv[r][j] != 0.0f) {
        if (pos < cap) {
          idx_out[pos] = static_cast<int>(i + j + 1);
          val_out[pos] = sv[r][j];
          sv[r][j] = 0.0f;                                // sent: leaves the residual
          sent = true;
        } else {
          ++lost;                                         // over capacity: stays in the residual
        }
        ++pos;
      }
    if (acc && sent) store4(acc, i, n, vec, sv[r]);
  }
  if (lost) atomicAdd(dropped, static_cast<unsigned long long>(lost));
}

// ---------------------------------------------------------------- top-K mode
// mode 0 "magnitude": key = bits of |s| (monotonic in |s| for non-NaN);
// mode 1 "compat":    key = |(int)s|, the value the reference's comparator
//                     actually compares (both operands truncated to int).
__device__ __forceinline__ unsigned make_key(float s, int mode) {
  if (mode == 0) return __float_as_uint(s) & 0x7fffffffu;
  const int t = static_cast<int>(s);  // saturating truncation toward zero
  return t < 0 ? 0u - static_cast<unsigned>(t) : static_cast<unsigned>(t);
}

// Pass p (0,1,2) histograms bits [20..31], [10..19], [0..9] of the keys whose
// higher bits equal the prefix decided so far.  Pass 0 also materialises
// s = g + acc into `sum` so later passes read 4 bytes per element.
template <int PASS>
__global__ void __launch_bounds__(kBlock)
topk_hist_kernel(const float* __restrict__ g, const float* __restrict__ acc,
                 float* __restrict__ sum, size_t n, int mode,
                 const SelectState* __restrict__ st, unsigned* __restrict__ hist, bool vec) {
  constexpr int kBins = PASS == 0 ? kBins1 : kBins23;
  constexpr int kShift = PASS == 0 ? 20 : (PASS == 1 ? 10 : 0);
  __shared__ unsigned sh[kBins];
  if (PASS == 1 && st->skip1) return;               // uniform for the whole grid
  for (int b = threadIdx.x; b < kBins; b += kBlock) sh[b] = 0;
  __syncthreads();
  unsigned top = 0;                                  // PASS 0: largest key of this thread
  const unsigned prefix = PASS == 0 ? 0u : st->prefix;
  const unsigned hi_mask = PASS == 0 ? 0u : (PASS == 1 ? 0xfff00000u : 0xfffffc00u);
  for (size_t tile = blockIdx.x; tile * kTile < n; tile += gridDim.x) {
    const size_t base = tile * kTile;
#pragma unroll
    for (int r = 0; r < kVecPerThread; ++r) {
      const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
      float s[4];
      if (PASS == 0) {
        load_sum4(g, acc, i, n, vec, s);
        if (acc) store4(sum, i, n, vec, s);         // sum == acc: the residual buffer now holds g + acc
      } else {
        load_sum4(sum, nullptr, i, n, vec, s);
      }
      unsigned bin[4];
      bool take[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned key = make_key(s[j], mode);
        take[j] = i + j < n && (key & hi_mask) == prefix;
        bin[j] = (key >> kShift) & (kBins - 1);
        if (PASS == 0 && i + j < n) top = max(top, key);
      }
      // Fast path: every lane of the warp takes all four of its elements and
      // they all fall into one bin (always true when every key ties): one
      // shared-memory atomic per warp for 128 elements.
      const bool mine_same = take[0] && take[1] && take[2] && take[3] && bin[0] == bin[1] &&
                             bin[1] == bin[2] && bin[2] == bin[3];
      const unsigned b0 = __shfl_sync(0xffffffffu, bin[0], 0);
      if (__all_sync(0xffffffffu, mine_same && bin[0] == b0)) {
        if ((threadIdx.x & 31) == 0) atomicAdd(&sh[b0], 128u);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (take[j]) atomicAdd(&sh[bin[j]], 1u);
      }
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < kBins; b += kBlock)
    if (sh[b]) atomicAdd(&hist[b], sh[b]);
  if (PASS == 0) {
    top = __reduce_max_sync(0xffffffffu, top);
    if ((threadIdx.x & 31) == 0 && top) atomicMax(const_cast<unsigned*>(&st->max_key), top);
  }
}

// One CTA: find the bin, counted from the top, in which the cumulative count
// reaches `remaining`, and fix that bin's bits into the prefix.  Each of the
// 1024 threads owns kBins/1024 consecutive bins (descending), a block-wide
// inclusive scan gives every thread the count of all higher bins, and exactly
// one thread finds the crossing inside its own bins.  Clears the histogram for
// the next pass.
template <int PASS>
__global__ void __launch_bounds__(1024)
topk_pick_kernel(unsigned* __restrict__ hist, SelectState* __restrict__ st, unsigned k_total) {
  constexpr int kBins = PASS == 0 ? kBins1 : kBins23;
  constexpr int kShift = PASS == 0 ? 20 : (PASS == 1 ? 10 : 0);
  constexpr int kPer = kBins / 1024;                 // 4 or 1 bins per thread
  __shared__ unsigned warp_tot[32];
  if (PASS == 1 && st->skip1) return;                // prefix and remaining stand; the histogram is still clear
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  // thread t owns descending bins  kBins-1 - t*kPer - j,  j = 0 .. kPer-1
  unsigned mine[kPer], local = 0;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int b = kBins - 1 - (threadIdx.x * kPer + j);
    mine[j] = hist[b];
    hist[b] = 0;
    local += mine[j];
  }
  unsigned incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned u = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += u;
  }
  if (lane == 31) warp_tot[w] = incl;
  __syncthreads();
  if (w == 0) {
    const unsigned t = warp_tot[lane];
    unsigned x = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned u = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += u;
    }
    warp_tot[lane] = x - t;                          // exclusive over warps
  }
  __syncthreads();
  const unsigned remaining0 = PASS == 0 ? k_total : st->remaining;
  const unsigned prefix0 = PASS == 0 ? 0u : st->prefix;
  unsigned above = warp_tot[w] + incl - local;       // elements in bins above this thread's
  __syncthreads();
  // crossing thread: above < remaining0 <= above + local.  If the total is
  // short (cannot happen for k <= n) the lowest bin takes whatever is left.
  const bool last = threadIdx.x == 1023;
  if (above < remaining0 && (remaining0 <= above + local || last)) {
    unsigned remaining = remaining0 - above;
    int b = kBins - 1 - threadIdx.x * kPer;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      if (mine[j] >= remaining || (last && j == kPer - 1)) break;
      remaining -= mine[j];
      --b;
    }
    const unsigned prefix = prefix0 | (static_cast<unsigned>(b) << kShift);
    st->prefix = prefix;
    st->remaining = remaining;
    // Keys that all fit in the lowest digit (the integer-truncated keys of small
    // gradients) leave the middle digit zero everywhere: skip that pass.
    if (PASS == 0) st->skip1 = st->max_key < (1u << 10) ? 1u : 0u;
    if (PASS == 2) {
      st->threshold = prefix;
      st->quota = remaining;
      st->nnz = static_cast<int>(k_total);
    }
  }
}

__global__ void __launch_bounds__(kBlock)
topk_count_kernel(const float* __restrict__ sum, size_t n, int mode,
                  const SelectState* __restrict__ st, unsigned* __restrict__ tile_gt,
                  unsigned* __restrict__ tile_eq, bool vec) {
  __shared__ unsigned sg[8], se[8];
  const unsigned T = st->threshold;
  const size_t base = static_cast<size_t>(blockIdx.x) * kTile;
  unsigned gt = 0, eq = 0;
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    float s[4];
    load_sum4(sum, nullptr, i, n, vec, s);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i + j < n) {
        const unsigned key = make_key(s[j], mode);
        gt += key > T;
        eq += key == T;
      }
  }
  gt = __reduce_add_sync(0xffffffffu, gt);
  eq = __reduce_add_sync(0xffffffffu, eq);
  if ((threadIdx.x & 31) == 0) { sg[threadIdx.x >> 5] = gt; se[threadIdx.x >> 5] = eq; }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned a = 0, b = 0;
    for (int k = 0; k < 8; ++k) { a += sg[k]; b += se[k]; }
    tile_gt[blockIdx.x] = a;
    tile_eq[blockIdx.x] = b;
  }
}

// Selected: key > T, or key == T and fewer than `quota` equal keys precede it.
// Payload position = (#greater before) + min(#equal before, quota).
__global__ void __launch_bounds__(kBlock)
topk_write_kernel(const float* __restrict__ sum, float* __restrict__ acc, size_t n, int mode,
                  const SelectState* __restrict__ st, const unsigned* __restrict__ gt_off,
                  const unsigned* __restrict__ eq_off, int* __restrict__ idx_out,
                  float* __restrict__ val_out, bool vec) {
  __shared__ unsigned sm[33];
  const unsigned T = st->threshold, quota = st->quota;
  // A tile that holds no key above T and no key == T that is still within the
  // quota sends nothing, and its residual (acc already holds g + acc) stays as
  // it is: leave before reading a byte.  The counts are differences of the
  // scanned offsets; the last tile has no successor and always runs.
  if (blockIdx.x + 1 < gridDim.x) {
    const unsigned g_lo = gt_off[blockIdx.x], e_lo = eq_off[blockIdx.x];
    const unsigned n_gt = gt_off[blockIdx.x + 1] - g_lo, n_eq = eq_off[blockIdx.x + 1] - e_lo;
    if (n_gt == 0 && (n_eq == 0 || e_lo >= quota)) return;
  }
  const size_t base = static_cast<size_t>(blockIdx.x) * kTile;
  float s[kVecPerThread][4];
  unsigned cg[kVecPerThread], ce[kVecPerThread], eg[kVecPerThread], ee[kVecPerThread];
  unsigned char flag[kVecPerThread][4];  // 0 none, 1 greater, 2 equal
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    cg[r] = 0; ce[r] = 0;
    load_sum4(sum, nullptr, i, n, vec, s[r]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      flag[r][j] = 0;
      if (i + j < n) {
        const unsigned key = make_key(s[r][j], mode);
        if (key > T) { flag[r][j] = 1; ++cg[r]; }
        else if (key == T) { flag[r][j] = 2; ++ce[r]; }
      }
    }
  }
  {  // one scan for both counters: greater in the high half, equal in the low half (each <= 4096)
    unsigned packed[kVecPerThread], excl[kVecPerThread];
#pragma unroll
    for (int r = 0; r < kVecPerThread; ++r) packed[r] = (cg[r] << 16) | ce[r];
    tile_exclusive(packed, excl, sm);
#pragma unroll
    for (int r = 0; r < kVecPerThread; ++r) {
      eg[r] = excl[r] >> 16;
      ee[r] = excl[r] & 0xffffu;
    }
  }
  const unsigned g0 = gt_off[blockIdx.x], e0 = eq_off[blockIdx.x];
#pragma unroll
  for (int r = 0; r < kVecPerThread; ++r) {
    const size_t i = base + (static_cast<size_t>(r) * kBlock + threadIdx.x) * 4;
    unsigned ng = g0 + eg[r], ne = e0 + ee[r];
    float res[4];
    bool any = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      bool sel = false;
      if (flag[r][j] == 1) {
        sel = true;
      } else if (flag[r][j] == 2) {
        sel = ne < quota;
      }
      if (sel) {
        const unsigned pos = ng + (ne < quota ? ne : quota);
        idx_out[pos] = static_cast<int>(i + j + 1);
        val_out[pos] = s[r][j];
      }
      res[j] = sel ? 0.0f : s[r][j];  // s - s == 0 when sent
      any = any || sel;
      if (flag[r][j] == 1) ++ng;
      if (flag[r][j] == 2) ++ne;
    }
    if (acc && any) store4(acc, i, n, vec, res);     // acc already holds s everywhere else
  }
}

// ------------------------------------------------------------- scatter-add
// dst[idx-1] += val for one rank's payload; the count lives on the device when
// count_dev != NULL (entry `rank_slot`), else `count` is used.  Index 0 marks
// padding and is skipped; indices are unique within a payload, so there are
// no conflicting updates inside one launch.
__global__ void __launch_bounds__(kBlock)
scatter_add_kernel(const int* __restrict__ idx, const float* __restrict__ val, size_t count,
                   const int* __restrict__ count_dev, float* __restrict__ dst, size_t n) {
  size_t m = count;
  if (count_dev) {                                  // the host count is then the capacity of idx / val
    const int dv = *count_dev;
    const size_t d = dv > 0 ? static_cast<size_t>(dv) : 0;
    m = d < count ? d : count;
  }
  for (size_t j = blockIdx.x * static_cast<size_t>(kBlock) + threadIdx.x; j < m;
       j += static_cast<size_t>(gridDim.x) * kBlock) {
    const int i = idx[j];
    if (i > 0 && static_cast<size_t>(i) <= n) dst[i - 1] += val[j];
  }
}

int check_common(const float* g, size_t n, const void* idx_out, const void* val_out, void* ws,
                 size_t ws_bytes) {
  if (!g || !idx_out || !val_out) return SGB_ERR_NULL;
  if (n > 0x7fffffffu) return SGB_ERR_SIZE;  // 1-based int32 indices on the wire
  if (!ws || ws_bytes < workspace_bytes(n) || (reinterpret_cast<uintptr_t>(ws) & 255u))
    return SGB_ERR_WORKSPACE;
  return SGB_OK;
}

}  // namespace

// ---- two-phase form used by the communicator (declared in sparse.cuh) ------
int sparse_threshold_count(const float* g, float* acc, size_t n, float thr, int* nnz_dev,
                           void* ws, size_t ws_bytes, cudaStream_t s) {
  if (n == 0) {
    cudaError_t e = cudaMemsetAsync(nnz_dev, 0, sizeof(int), s);
    return e == cudaSuccess ? SGB_OK : note_cuda_error(e);
  }
  if (n > 0x7fffffffu) return SGB_ERR_SIZE;
  if (!ws || ws_bytes < workspace_bytes(n) || (reinterpret_cast<uintptr_t>(ws) & 255u))
    return SGB_ERR_WORKSPACE;
  Workspace w = carve(ws, n);
  const unsigned tiles = static_cast<unsigned>(tiles_of(n));
  thr_count_kernel<<<tiles, kBlock, 0, s>>>(g, acc, n, thr, w.tile_counts, aligned16(g) && (!acc || aligned16(acc)));
  scan_tiles_kernel<<<1, 1024, 0, s>>>(w.tile_counts, nullptr, tiles, w.state, 1);
  cudaError_t e = cudaMemcpyAsync(nnz_dev, &w.state->nnz, sizeof(int), cudaMemcpyDeviceToDevice, s);
  if (e != cudaSuccess) return note_cuda_error(e);
  return launch_status();
}

int sparse_threshold_write_packed(const float* g, float* acc, size_t n, float thr, int* payload,
                                  void* ws, cudaStream_t s) {
  if (n == 0) return SGB_OK;
  Workspace w = carve(ws, n);
  const unsigned tiles = static_cast<unsigned>(tiles_of(n));
  thr_write_kernel<<<tiles, kBlock, 0, s>>>(acc ? acc : g, acc, n, thr, w.tile_counts, payload, nullptr, w.state, aligned16(g) && (!acc || aligned16(acc)));
  return launch_status();
}

int sparse_threshold_write_bounded(const float* g, float* acc, size_t n, float thr, int* payload, size_t cap,
                                   unsigned long long* dropped_dev, void* ws, cudaStream_t s) {
  if (n == 0) return SGB_OK;
  if (cap == 0 || cap > 0x7fffffffu || !dropped_dev) return SGB_ERR_SIZE;
  Workspace w = carve(ws, n);
  const unsigned tiles = static_cast<unsigned>(tiles_of(n));
  thr_write_bounded_kernel<<<tiles, kBlock, 0, s>>>(acc ? acc : g, acc, n, thr, w.tile_counts, payload,
                                                    static_cast<unsigned>(cap), dropped_dev,
                                                    aligned16(g) && (!acc || aligned16(acc)));
  return launch_status();
}

}  // namespace sgb

using namespace sgb;

extern "C" {

size_t sgb_sparse_workspace_bytes(size_t n) { return n ? workspace_bytes(n) : 256; }

int sgb_topk_count(float ratio, size_t n) {
  // (int)ceil(threshold * num) evaluated in fp32, as the reference does
  // (float * size_t -> float).
  const float prod = ratio * static_cast<float>(n);
  float c = ceilf(prod);
  if (c < 0.f) c = 0.f;
  if (c > static_cast<float>(n)) return static_cast<int>(n);
  return static_cast<int>(c);
}

int sgb_sparse_threshold_f32(const float* g, float* acc, size_t n, float thr, int32_t* idx_out,
                             float* val_out, int32_t* nnz_dev, void* ws, size_t ws_bytes,
                             void* stream) {
  if (!nnz_dev) return SGB_ERR_NULL;
  cudaStream_t s = as_stream(stream);
  if (n == 0) {
    cudaError_t e = cudaMemsetAsync(nnz_dev, 0, sizeof(int), s);
    return e == cudaSuccess ? SGB_OK : note_cuda_error(e);
  }
  int st = check_common(g, n, idx_out, val_out, ws, ws_bytes);
  if (st != SGB_OK) return st;
  Workspace w = carve(ws, n);
  const unsigned tiles = static_cast<unsigned>(tiles_of(n));
  thr_count_kernel<<<tiles, kBlock, 0, s>>>(g, acc, n, thr, w.tile_counts, aligned16(g) && (!acc || aligned16(acc)));
  scan_tiles_kernel<<<1, 1024, 0, s>>>(w.tile_counts, nullptr, tiles, w.state, 1);
  cudaError_t e = cudaMemcpyAsync(nnz_dev, &w.state->nnz, sizeof(int), cudaMemcpyDeviceToDevice, s);
  if (e != cudaSuccess) return note_cuda_error(e);
  thr_write_kernel<<<tiles, kBlock, 0, s>>>(acc ? acc : g, acc, n, thr, w.tile_counts, idx_out, val_out, w.state, aligned16(g) && (!acc || aligned16(acc)));
  return launch_status();
}

int sgb_sparse_topk_f32(const float* g, float* acc, float* sum_scratch, size_t n, size_t k,
                        int mode, int32_t* idx_out, float* val_out, void* ws, size_t ws_bytes,
                        void* stream) {
  if (n == 0 || k == 0) return SGB_OK;
  if (mode != 0 && mode != 1) return SGB_ERR_UNSUPPORTED;
  (void)sum_scratch;   // kept in the signature; the sum lives in acc (or is g itself without a residual)
  int st = check_common(g, n, idx_out, val_out, ws, ws_bytes);
  if (st != SGB_OK) return st;
  if (k > n) k = n;
  cudaStream_t s = as_stream(stream);
  Workspace w = carve(ws, n);
  const unsigned tiles = static_cast<unsigned>(tiles_of(n));
  const unsigned hgrid = capped_grid(tiles, 1, 8);
  const bool vec = aligned16(g) && (!acc || aligned16(acc));
  float* sum = acc ? acc : const_cast<float*>(g);
  // histogram and the selection state behind it (one contiguous region)
  cudaError_t e = cudaMemsetAsync(w.hist, 0, align256(kBins1 * sizeof(unsigned)) + sizeof(SelectState), s);
  if (e != cudaSuccess) return note_cuda_error(e);
  topk_hist_kernel<0><<<hgrid, kBlock, 0, s>>>(g, acc, sum, n, mode, w.state, w.hist, vec);
  topk_pick_kernel<0><<<1, 1024, 0, s>>>(w.hist, w.state, static_cast<unsigned>(k));
  topk_hist_kernel<1><<<hgrid, kBlock, 0, s>>>(g, acc, sum, n, mode, w.state, w.hist, vec);
  topk_pick_kernel<1><<<1, 1024, 0, s>>>(w.hist, w.state, static_cast<unsigned>(k));
  topk_hist_kernel<2><<<hgrid, kBlock, 0, s>>>(g, acc, sum, n, mode, w.state, w.hist, vec);
  topk_pick_kernel<2><<<1, 1024, 0, s>>>(w.hist, w.state, static_cast<unsigned>(k));
  topk_count_kernel<<<tiles, kBlock, 0, s>>>(sum, n, mode, w.state, w.tile_gt, w.tile_eq, vec);
  scan_tiles_kernel<<<1, 1024, 0, s>>>(w.tile_gt, w.tile_eq, tiles, w.state, 0);
  topk_write_kernel<<<tiles, kBlock, 0, s>>>(sum, acc, n, mode, w.state, w.tile_gt,
                                             w.tile_eq, idx_out, val_out, vec);
  return launch_status();
}

int sgb_scatter_add_f32(const int32_t* idx, const float* val, size_t count,
                        const int32_t* count_dev, float* dst, size_t n, void* stream) {
  if (!count_dev && count == 0) return SGB_OK;
  if (!idx || !val || !dst) return SGB_ERR_NULL;
  const size_t guess = count_dev ? (count ? count : n) : count;
  unsigned grid = capped_grid(guess, kBlock, 8);
  scatter_add_kernel<<<grid, kBlock, 0, as_stream(stream)>>>(idx, val, count, count_dev, dst, n);
  return launch_status();
}

}  // extern "C"
