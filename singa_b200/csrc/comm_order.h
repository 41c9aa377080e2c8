// Host-only: which cross-stream edges each communicator call records.
//
// The communicator works on four streams: the caller's compute stream, c1
// (pre-processing: pack, cast down, select), s (NCCL) and c2 (post-processing:
// cast up, unpack of fp16 buckets, scatter-add).  This file is the single
// statement of the ordering rules; comm.cu emits exactly the edges planned
// here, and the planner is exported (sgb_comm_order_plan) so that the rules
// can be replayed over a whole step on a machine without a GPU.
//
// Rules (the reference records its event on the compute stream before EVERY
// stage and flush, src/io/communicator.cc:227-233, 255-271, 313-319):
//   * every collective is ordered after the compute stream at the point of the
//     call: directly (compute -> s) when it reads the caller's tensors in
//     place, through c1 (compute -> c1 -> s) when a kernel on c1 packs, casts
//     or selects first;
//   * a collective that writes a communicator-owned receive buffer is ordered
//     after the last kernel on c2 that read such a buffer (event recorded
//     right behind that kernel, so later work on c2 does not delay NCCL);
//   * the stream that post-processes, or on which a caller may consume the
//     result, waits for the collective (s -> c1 / s -> c2);
//   * wait() joins every stream that received work back to the compute stream.
#pragma once

namespace sgb {
namespace order {

enum Call {
  kSynch = 0,         // one tensor, all-reduced in place
  kFlushInPlace = 1,  // a bucket whose tensors lie back to back: reduced in place
  kFlushPacked = 2,   // pack on c1, all-reduce send -> recv, unpack on c1
  kFlushHalf = 3,     // pack + cast on c1, fp16 all-reduce, cast + unpack on c2
  kSynchHalf = 4,     // cast on c1, fp16 all-reduce, cast back on c2
  kSparse = 5,        // select on c1, all-gather, scatter-add on c2
  kStageCopy = 6,     // copies into the staging buffer on c1 (no collective)
  kWait = 7,
};

enum Edge : unsigned {
  kComputeToC1 = 1u << 0,
  kComputeToS = 1u << 1,
  kC1ToS = 1u << 2,
  kC2DoneToS = 1u << 3,   // s waits for the event recorded behind the last post-processing kernel
  kSToC1 = 1u << 4,
  kSToC2 = 1u << 5,
  kSToCompute = 1u << 6,
  kC1ToCompute = 1u << 7,
  kC2ToCompute = 1u << 8,
  kMarkC2Done = 1u << 9,  // record that event on c2
};

enum { kStreamS = 0, kStreamC1 = 1, kStreamC2 = 2 };

struct State {
  unsigned char dirty_s = 0, dirty_c1 = 0, dirty_c2 = 0;  // received work since the last wait()
  unsigned char c2_reads_recv = 0;  // a kernel on c2 read a receive buffer since s last waited for c2
};

struct Step {
  unsigned pre = 0;     // before the pre-processing kernel on c1
  unsigned before = 0;  // before the collective on s
  unsigned after = 0;   // behind the collective
  unsigned post = 0;    // behind the post-processing kernel
  int result_stream = kStreamS;  // where the reduced values can be consumed
};

inline Step plan(State& st, int call) {
  Step p;
  switch (call) {
    case kSynch:
    case kFlushInPlace:
      p.before = kComputeToS;
      p.after = kSToC2;
      p.result_stream = kStreamC2;
      st.dirty_s = st.dirty_c2 = 1;
      break;
    case kFlushPacked:
      p.pre = kComputeToC1;
      p.before = kC1ToS | (st.c2_reads_recv ? kC2DoneToS : 0u);
      p.after = kSToC1;
      p.result_stream = kStreamC1;
      st.c2_reads_recv = 0;
      st.dirty_s = st.dirty_c1 = 1;
      break;
    case kFlushHalf:
    case kSynchHalf:
    case kSparse:
      p.pre = kComputeToC1;
      p.before = kC1ToS | (st.c2_reads_recv ? kC2DoneToS : 0u);
      p.after = kSToC1 | kSToC2;
      p.post = kMarkC2Done;
      p.result_stream = kStreamC2;
      st.c2_reads_recv = 1;
      st.dirty_s = st.dirty_c1 = st.dirty_c2 = 1;
      break;
    case kStageCopy:
      p.pre = kComputeToC1;
      p.result_stream = kStreamC1;
      st.dirty_c1 = 1;
      break;
    case kWait:
      p.before = (st.dirty_s ? kSToCompute : 0u) | (st.dirty_c1 ? kC1ToCompute : 0u) |
                 (st.dirty_c2 ? kC2ToCompute : 0u);
      st = State();
      break;
    default:
      break;
  }
  return p;
}

}  // namespace order
}  // namespace sgb
