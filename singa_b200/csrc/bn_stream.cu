// Batch-norm backward as a persistent streaming kernel (single pass over HBM,
// 12 bytes per element; 16 with the ReLU input as floats).
//
// Work is cut into items: S consecutive pieces of one channel (a piece is a
// contiguous run of Lp floats inside one sample's plane), about 50 KB of x and
// dy.  Small CTAs (128 threads, one staging slot each, three to sixteen per
// SM) take items from a device-wide ticket counter until none is left.  Per
// item a CTA
//   1. brings the pieces of x / dy (/ ReLU input or bit record) into its slot
//      with bulk asynchronous copies (cp.async.bulk, completion counted on an
//      mbarrier);
//   2. forms the item's two partial sums (sum dy, sum dy * (x - mean)) and
//      publishes them: the pair goes to the workspace, then the channel's
//      counter in global memory is incremented (release);
//   3. polls that counter until every item of the channel has published
//      (bounded), then adds all pairs in item order - every CTA forms the same
//      totals, so results do not depend on timing;
//   4. turns the staged x into dx in place and writes the pieces back with bulk
//      copies; while they drain it already holds its next ticket.
// The CTAs of an SM are at different steps at any moment, so the SM always has
// copies in flight; nothing depends on how CTAs are placed (no cluster), every
// SM slot is used, and no CTA is launched or retired between items.
//
// Tickets are handed out in item order and only to running CTAs, and a CTA
// draws its next ticket only after its current item no longer waits for
// anybody, so an item never waits for a CTA that is not resident or for an
// item that nobody can load.  The counters live in a table inside the library
// (zero when idle; every launch leaves its table zero again); the host hands
// tables out round robin and the kernel checks that its table is not in use by
// another launch.
//
// Every wait is bounded by a deadline; when one runs out the CTA sets a sticky
// fault word (bn_stream_faults), stops taking items, waits for its copies in
// flight and returns.
#include "bn_stream.cuh"

#include <atomic>

#include "bulk_copy.cuh"
#include "common.cuh"

namespace sgb {
namespace {

constexpr int kThreads = 128;
constexpr int kMaxCtasPerSm = 16;
constexpr int kTables = 8;
constexpr int kMaxChannels = 4096;
constexpr int kSlotTarget = 25088;               // bytes of one staged tensor per item (2 planes of 56 x 56)
constexpr int kSmemBudget = 225 * 1024;
constexpr unsigned long long kDeadlineTicks = 8000000000ull;   // about 4 s at 2 GHz
constexpr unsigned kFaultTimeout = 1u, kFaultTableBusy = 2u;

struct ExchangeTable {
  unsigned next_item;                 // ticket counter
  unsigned finished;                  // CTAs of the launch that have returned
  unsigned owner;                     // tag of the launch using the table, 0 = idle
  unsigned pad;
  unsigned arrived[kMaxChannels];     // per channel: items published + CTAs that have read the totals
};
__device__ ExchangeTable g_tables[kTables];
__device__ unsigned g_faults;

struct Tail {                         // shared memory behind the slot
  unsigned long long full;            // the item's copies have landed
  int item;                           // the CTA's next ticket
  int abort;
  float sums[2];                      // the channel's totals
  float red[2][kThreads / 32];
};

struct StreamArgs {
  const float* x;
  const float* dy;
  const void* relu;
  const float* scale;
  const float* mean;
  const float* invstd;
  float* dx;
  float* dscale;
  float* dbias;
  float2* partial;
  int N, C, HW;
  int P, Lp, S, parts, depth;
  int pieces;        // N * P pieces per channel
  int items;         // C * parts
  int slot_bytes;    // whole slot
  int mask_stride;   // bytes reserved per piece for the bit record (mask 2)
  int table;
  unsigned tag;
};

// Deadlines are counted in SM clock cycles (a plain register read, local to
// the SM the CTA runs on).
__device__ __forceinline__ unsigned long long now_ticks() { return static_cast<unsigned long long>(clock64()); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Polls an mbarrier phase until it completes, the CTA aborts or the deadline passes.
__device__ __forceinline__ bool wait_phase(unsigned long long* bar, unsigned parity, volatile int* abort,
                                           unsigned long long deadline) {
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 15u) == 0) {
      if (*abort) return false;
      if (now_ticks() > deadline) {
        *abort = 1;
        atomicOr(&g_faults, kFaultTimeout);
        return false;
      }
    }
  }
}

// Position of an item's piece q in global memory (floats from the tensor base).
__device__ __forceinline__ size_t piece_offset(const StreamArgs& a, int c, int piece) {
  const int n = piece / a.P, r = piece - n * a.P;
  return (static_cast<size_t>(n) * a.C + c) * a.HW + static_cast<size_t>(r) * a.Lp;
}

// Bytes [lo, hi) of the bit record that a piece starting at element e0 needs,
// widened to 16-byte boundaries (the record is allocated in 16-byte groups).
__device__ __forceinline__ void record_span(size_t e0, int Lp, size_t* lo, unsigned* bytes) {
  const size_t first = (e0 >> 3) & ~static_cast<size_t>(15);
  const size_t last = (((e0 + Lp + 7) >> 3) + 15) & ~static_cast<size_t>(15);
  *lo = first;
  *bytes = static_cast<unsigned>(last - first);
}

// Polls a counter in global memory until it reaches `want`, the CTA aborts or
// the deadline passes.
__device__ __forceinline__ bool poll_counter(const unsigned* ctr, unsigned want, volatile int* abort,
                                             unsigned long long deadline) {
  for (unsigned it = 1;; ++it) {
    if (ld_acquire(ctr) >= want) return true;
    if ((it & 7u) == 0) {
      if (*abort) return false;
      if (now_ticks() > deadline) {
        *abort = 1;
        atomicOr(&g_faults, kFaultTimeout);
        return false;
      }
    }
    if (it > 4) __nanosleep(32);
  }
}

template <int MASK>
__global__ void __launch_bounds__(kThreads) bn_bwd_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* slot = smem;
  Tail* tail = reinterpret_cast<Tail*>(smem + a.slot_bytes);
  ExchangeTable& tab = g_tables[a.table];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort = &tail->abort;
  if (tid == 0) {
    mbar_init(&tail->full, 1);
    tail->abort = 0;
    fence_mbarrier_init();
    dependency_wait();                                // first access to global memory follows
    // both requests travel together; a ticket drawn from a table that turns
    // out to be another launch's is reported as a fault (both launches are void)
    const unsigned old = atomicCAS(&tab.owner, 0u, a.tag);
    const unsigned first = atomicAdd(&tab.next_item, 1u);
    if (old != 0u && old != a.tag) {                  // the table belongs to another launch still running
      atomicOr(&g_faults, kFaultTableBusy);
      tail->abort = 2;
    } else {
      tail->item = static_cast<int>(first);
    }
  }
  __syncthreads();
  dependency_wait();
  // The next kernel of the stream may be scheduled as soon as SM slots free up
  // (it waits for this grid to complete before it touches memory): every CTA
  // of this grid is running by the time all of them have said so.
  release_dependents();
  if (tail->abort == 2) return;                       // nothing was issued, nothing of the table was touched
  const unsigned long long deadline = now_ticks() + kDeadlineTicks;
  const int array_floats = a.S * a.Lp;                // floats of one staged tensor in the slot
  const unsigned piece_bytes = static_cast<unsigned>(a.Lp) * 4u;
  const int upp = a.Lp / 4;                           // 16-byte units per piece
  const float inv_m = 1.0f / (static_cast<float>(a.N) * static_cast<float>(a.HW));
  constexpr int kWarps = kThreads / 32;
  float* sx = reinterpret_cast<float*>(slot);
  float* sg = sx + array_floats;

  int t = *reinterpret_cast<volatile int*>(&tail->item);
  unsigned use = 0;
  bool gave_up = false;
  while (t < a.items) {
    const int c = t / a.parts, p = t - c * a.parts;
    const int p0 = p * a.S, np = min(a.S, a.pieces - p0);
    if (warp == 0) {
      // bring the item in: one bulk copy per piece and tensor, counted on `full`
      unsigned bytes = (MASK == 1 ? 3u : 2u) * static_cast<unsigned>(np) * piece_bytes;
      if (MASK == 2) {
        unsigned mine = 0;
        for (int q = lane; q < np; q += 32) {
          size_t lo;
          unsigned nb;
          record_span(piece_offset(a, c, p0 + q), a.Lp, &lo, &nb);
          mine += nb;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        bytes += mine;
      }
      if (lane == 0) mbar_arrive_expect(&tail->full, bytes);
      __syncwarp();
      for (int q = lane; q < np; q += 32) {
        const size_t off = piece_offset(a, c, p0 + q);
        float* dst = sx + static_cast<size_t>(q) * a.Lp;
        bulk_load(dst, a.x + off, piece_bytes, &tail->full);
        bulk_load(dst + array_floats, a.dy + off, piece_bytes, &tail->full);
        if (MASK == 1)
          bulk_load(dst + 2 * array_floats, static_cast<const float*>(a.relu) + off, piece_bytes, &tail->full);
        if (MASK == 2) {
          size_t lo;
          unsigned nb;
          record_span(off, a.Lp, &lo, &nb);
          bulk_load(slot + static_cast<size_t>(2) * array_floats * 4 + static_cast<size_t>(q) * a.mask_stride,
                    static_cast<const unsigned char*>(a.relu) + lo, nb, &tail->full);
        }
      }
    }
    // the channel's constants arrive while the copies fly
    const float mu = __ldg(a.mean + c), r_ = __ldg(a.invstd + c), sc = __ldg(a.scale + c);
    const bool landed = wait_phase(&tail->full, use & 1u, abort, deadline);
    if (__syncthreads_or(landed ? 0 : 1)) {
      gave_up = true;
      break;
    }

    // ---- the item's pair: sum dy, sum dy * (x - mean)
    const int units = np * upp;
    float s_dy = 0.f, s_dyx = 0.f;
    for (int u = tid; u < units; u += kThreads) {
      Vec4f vx, vg;
      vx.u = *reinterpret_cast<const uint4*>(sx + 4 * u);
      vg.u = *reinterpret_cast<const uint4*>(sg + 4 * u);
      if (MASK == 1) {
        Vec4f vr;
        vr.u = *reinterpret_cast<const uint4*>(sg + array_floats + 4 * u);
#pragma unroll
        for (int q = 0; q < 4; ++q) vg.f[q] = vr.f[q] > 0 ? vg.f[q] : 0.0f;
        *reinterpret_cast<uint4*>(sg + 4 * u) = vg.u;          // the masked gradient, for the second pass
      }
      if (MASK == 2) {
        const int q = u / upp, r = u - q * upp;
        // the piece's record was copied from a 16-byte boundary: its first bit is bit (e0 mod 128)
        const unsigned e0 = static_cast<unsigned>(piece_offset(a, c, p0 + q));
        const unsigned bit = (e0 & 127u) + 4u * static_cast<unsigned>(r);
        const unsigned char rec =
            slot[static_cast<size_t>(2) * array_floats * 4 + static_cast<size_t>(q) * a.mask_stride + (bit >> 3)];
        const unsigned keep = (rec >> (bit & 4u)) & 15u;
#pragma unroll
        for (int j = 0; j < 4; ++j) vg.f[j] = (keep >> j) & 1u ? vg.f[j] : 0.0f;
        *reinterpret_cast<uint4*>(sg + 4 * u) = vg.u;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        s_dy += vg.f[q];
        s_dyx += vg.f[q] * (vx.f[q] - mu);
      }
    }
    s_dy = warp_sum(s_dy);
    s_dyx = warp_sum(s_dyx);
    if (lane == 0) {
      tail->red[0][warp] = s_dy;
      tail->red[1][warp] = s_dyx;
    }
    __syncthreads();

    // ---- the channel's totals (warp 0), and the next ticket
    int bad = 0;
    if (warp == 0) {
      float ta = lane < kWarps ? tail->red[0][lane] : 0.0f;
      float tb = lane < kWarps ? tail->red[1][lane] : 0.0f;
      ta = warp_sum(ta);
      tb = warp_sum(tb);
      int next = a.items;
      if (a.parts > 1) {
        int good = 1;
        if (lane == 0) {
          // publish: the pair, then (release) one more arrival on the channel's counter
          __stcg(&a.partial[t], make_float2(ta, tb));
          asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(&tab.arrived[c]), "r"(1u) : "memory");
          good = poll_counter(&tab.arrived[c], static_cast<unsigned>(a.parts), abort, deadline) ? 1 : 0;
          // from here on this CTA only finishes its item: the next ticket can be drawn
          if (good) next = static_cast<int>(atomicAdd(&tab.next_item, 1u));
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        ta = 0.f;
        tb = 0.f;
        if (good) {
          for (int q = lane; q < a.parts; q += 32) {  // every CTA adds the pairs in the same order
            const float2 v = __ldcg(&a.partial[c * a.parts + q]);
            ta += v.x;
            tb += v.y;
          }
        }
        ta = warp_sum(ta);
        tb = warp_sum(tb);
        bad = good ? 0 : 1;
      } else if (lane == 0) {
        next = static_cast<int>(atomicAdd(&tab.next_item, 1u));
      }
      if (lane == 0) {
        tail->sums[0] = ta;
        tail->sums[1] = tb;
        tail->item = next;
      }
    }
    if (__syncthreads_or(bad)) {
      gave_up = true;
      break;
    }

    // ---- dx in place of x
    const float sum_dy = *reinterpret_cast<volatile float*>(&tail->sums[0]);
    const float sum_dyx = *reinterpret_cast<volatile float*>(&tail->sums[1]);
    const float ds = sum_dyx * r_;
    const float k_ = sc * r_, am = sum_dy * inv_m, bm = ds * r_ * inv_m;
    if (p == 0 && tid == 0) {
      a.dscale[c] = ds;
      a.dbias[c] = sum_dy;
    }
    for (int u = tid; u < units; u += kThreads) {
      Vec4f vx, vg, o;
      vx.u = *reinterpret_cast<const uint4*>(sx + 4 * u);
      vg.u = *reinterpret_cast<const uint4*>(sg + 4 * u);
#pragma unroll
      for (int j = 0; j < 4; ++j) o.f[j] = k_ * (vg.f[j] - am - (vx.f[j] - mu) * bm);
      *reinterpret_cast<uint4*>(sx + 4 * u) = o.u;
    }
    fence_async_smem();                               // the bulk copy engine reads what was just written
    __syncthreads();
    if (warp == 0) {
      for (int q = lane; q < np; q += 32)
        bulk_store(a.dx + piece_offset(a, c, p0 + q), sx + static_cast<size_t>(q) * a.Lp, piece_bytes);
      bulk_commit();
      if (a.parts > 1 && lane == 0) {
        // the last of the channel's readers leaves its counter at zero
        const unsigned old = atomicAdd(&tab.arrived[c], 1u);
        if (old == 2u * static_cast<unsigned>(a.parts) - 1u) atomicExch(&tab.arrived[c], 0u);
      }
      bulk_wait_read();                               // the engine has read the slot: it can be refilled
    }
    __syncthreads();
    t = *reinterpret_cast<volatile int*>(&tail->item);
    ++use;
  }

  if (gave_up && tid == 0) {
    // copies into the slot may still be landing: they must finish before the CTA's memory goes away
    const unsigned long long limit = now_ticks() + 2000000000ull;
    while (!mbar_try_wait(&tail->full, use & 1u) && now_ticks() < limit) {
    }
  }
  if (warp == 0) bulk_wait_all();
  if (tid == 0) {
    __threadfence();
    const unsigned done = atomicAdd(&tab.finished, 1u);
    if (done == gridDim.x - 1 && ld_acquire(&g_faults) == 0u) {
      tab.next_item = 0;                              // the table is idle (all zero) again
      tab.finished = 0;
      __threadfence();
      atomicExch(&tab.owner, 0u);
    }
  }
}

constexpr int round_up(int v, int m) { return (v + m - 1) / m * m; }

int slot_bytes_of(const BnStreamPlan& p, int mask, int* mask_stride) {
  *mask_stride = mask == 2 ? round_up((p.Lp + 7) / 8, 16) + 32 : 0;
  return round_up(p.arrays * p.S * p.Lp * 4 + p.S * *mask_stride, 128);
}

template <int MASK>
int launch_stream(const StreamArgs& args, cudaStream_t s) {
  auto kernel = bn_bwd_stream_kernel<MASK>;
  static std::atomic<bool> attr_set[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
  const bool tracked = dev >= 0 && dev < 64;
  if (!tracked || !attr_set[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (tracked) attr_set[dev].store(true, std::memory_order_release);
  }
  const int resident = sm_count() * args.depth;
  const int grid = args.items < resident ? args.items : resident;
  const size_t smem = static_cast<size_t>(args.slot_bytes) + sizeof(Tail);
  return launch_ex(kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), smem, s, 0, true, args);
}

}  // namespace

bool bn_stream_plan(int N, int C, int HW, int mask, BnStreamPlan* plan) {
  if (N < 1 || C < 1 || HW < 4 || HW % 4 != 0 || C > kMaxChannels) return false;
  BnStreamPlan p{};
  p.P = 1;
  while (HW % p.P != 0 || (HW / p.P) % 4 != 0 || (HW / p.P) * 4 > kSlotTarget) {
    if (++p.P > 64) return false;
  }
  p.Lp = HW / p.P;
  const long long pieces = static_cast<long long>(N) * p.P;
  if (pieces > 1 << 20) return false;
  p.S = kSlotTarget / (p.Lp * 4);
  if (p.S < 1) p.S = 1;
  if (p.S > pieces) p.S = static_cast<int>(pieces);
  // enough items for every SM to get several (shape-only rule: the partition,
  // and with it the order of the additions, does not depend on the mask mode)
  const long long want = 24LL * sm_count();
  while (p.S > 1 && C * ((pieces + p.S - 1) / p.S) < want && ((p.S + 1) / 2) * p.Lp * 4 >= 4096) p.S = (p.S + 1) / 2;
  p.parts = static_cast<int>((pieces + p.S - 1) / p.S);
  if (p.parts > 64) return false;                      // also bounds the workspace: 64 pairs per channel
  p.arrays = mask == 1 ? 3 : 2;
  int mask_stride = 0;
  const int slot = slot_bytes_of(p, mask, &mask_stride);
  // CTAs per SM: each takes its slot, the tail and 1 KB the system reserves, out of 228 KB
  p.depth = (228 * 1024) / (round_up(slot + static_cast<int>(sizeof(Tail)), 128) + 1024);
  if (p.depth > kMaxCtasPerSm) p.depth = kMaxCtasPerSm;
  if (p.depth < 2) return false;
  *plan = p;
  return true;
}

size_t bn_stream_workspace_bytes(int N, int C, int HW) {
  (void)N;
  (void)HW;
  return static_cast<size_t>(64) * C * sizeof(float2);
}

int bn_stream_backward(int mask, const float* x, const float* dy, const void* relu, const float* scale,
                       const float* mean, const float* invstd, float* dx, float* dscale, float* dbias,
                       int N, int C, int HW, const BnStreamPlan& plan, void* partial, cudaStream_t s) {
  static std::atomic<unsigned> next_tag{1};
  StreamArgs a{};
  a.x = x;
  a.dy = dy;
  a.relu = relu;
  a.scale = scale;
  a.mean = mean;
  a.invstd = invstd;
  a.dx = dx;
  a.dscale = dscale;
  a.dbias = dbias;
  a.partial = static_cast<float2*>(partial);
  a.N = N;
  a.C = C;
  a.HW = HW;
  a.P = plan.P;
  a.Lp = plan.Lp;
  a.S = plan.S;
  a.parts = plan.parts;
  a.depth = plan.depth;
  a.pieces = N * plan.P;
  a.items = C * plan.parts;
  a.slot_bytes = slot_bytes_of(plan, mask, &a.mask_stride);
  unsigned tag = next_tag.fetch_add(1, std::memory_order_relaxed);
  if (tag == 0) tag = next_tag.fetch_add(1, std::memory_order_relaxed);
  a.tag = tag;
  a.table = static_cast<int>(tag % kTables);
  switch (mask) {
    case 0: return launch_stream<0>(a, s);
    case 1: return launch_stream<1>(a, s);
    case 2: return launch_stream<2>(a, s);
    default: return SGB_ERR_UNSUPPORTED;
  }
}

int bn_stream_faults(unsigned* flags) {
  if (!flags) return SGB_ERR_NULL;
  cudaError_t e = cudaMemcpyFromSymbol(flags, g_faults, sizeof(unsigned));
  return e == cudaSuccess ? SGB_OK : note_cuda_error(e);
}

}  // namespace sgb
