// Data-parallel gradient communicator: dense all-reduce (direct and bucketed),
// fp16-compressed all-reduce, and sparsified all-gather (threshold / top-K with
// residual correction), one process per GPU over NCCL on NVLink / NVSwitch.
//
// It keeps the reference communicator's observable structure - a compute
// stream plus three side streams (c1: pre-processing, s: NCCL, c2:
// post-processing) chained by events, staging buffers of maxSize elements,
// sum semantics (the caller divides by the world size) - and replaces the
// per-tensor memcpy / cast / thrust / cuSPARSE passes around the collectives
// by the fused kernels of this library:
//   stage   = one multi-tensor pack (+ fp32->fp16 cast) launch per call
//   flush   = collective + one multi-tensor unpack (+ fp16->fp32 cast) launch
//   sparse  = residual + select + order-preserving compaction, radix select
//             instead of a full sort, one scatter-add launch per rank.
// Each cross-stream edge has its own event.  No kernel here touches another
// GPU's memory: remote data reaches local HBM through NCCL only.
#include <nccl.h>

#include <atomic>
#include <cstring>
#include <new>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include <string>

#include "comm_order.h"
#include "common.cuh"
#include "sparse.cuh"

namespace {
std::atomic<int> g_last_nccl_error{0};

int nccl_fail(ncclResult_t r) {
  g_last_nccl_error.store(static_cast<int>(r));
  return SGB_ERR_NCCL;
}
}  // namespace

#define CU(call)                                            \
  do {                                                      \
    cudaError_t e__ = (call);                               \
    if (e__ != cudaSuccess) return sgb::note_cuda_error(e__); \
  } while (0)
#define NC(call)                                   \
  do {                                             \
    ncclResult_t r__ = (call);                     \
    if (r__ != ncclSuccess) return nccl_fail(r__); \
  } while (0)
#define OK(call)                     \
  do {                               \
    int s__ = (call);                \
    if (s__ != SGB_OK) return s__;   \
  } while (0)

struct sgb_comm {
  int rank = 0, world = 1, device = 0;
  ncclComm_t nccl = nullptr;
  size_t max_elems = 0;
  float* send = nullptr;   // fusedSendBuff
  float* recv = nullptr;   // fusedRecvBuff
  __half* send_h = nullptr;    // staging bucket in fp16
  __half* recv_h = nullptr;
  __half* dsend_h = nullptr;   // direct (unbucketed) fp16 synch: never aliases a half-filled bucket
  __half* drecv_h = nullptr;
  // sparse path (allocated at first use)
  float* sum = nullptr;        // g + acc (backupBuff)
  int* pay_send = nullptr;     // [idx | val], 2 * max_elems words
  int* pay_recv = nullptr;     // world * 2 * max_elems words
  void* ws = nullptr;
  size_t ws_bytes = 0;
  int* nnz_dev = nullptr;      // [0] own count, [1 .. world] all ranks
  int* nnz_host = nullptr;     // pinned, world entries
  unsigned long long* dropped_dev = nullptr;   // entries the bounded threshold form left for later calls
  int topk_mode = 1;           // 1 = the reference comparator's key, 0 = |value|
  cudaStream_t s = nullptr, c1 = nullptr, c2 = nullptr;
  bool own_streams = true;     // false after sgb_comm_use_streams: the caller's streams are not destroyed
  cudaEvent_t ev_compute = nullptr, ev_c1 = nullptr, ev_s = nullptr, ev_c2 = nullptr,
              ev_c2_done = nullptr, ev_host = nullptr;
  size_t send_off = 0;         // elements staged since the last flush
  // Which side streams received work since the last wait() (only those are
  // joined, so a wait() issued while the compute stream is being captured
  // never touches a stream outside the capture) and whether c2 still reads a
  // receive buffer: the state of the edge planner in comm_order.h.
  sgb::order::State order;
  int result_stream = sgb::order::kStreamS;   // where the last call's result can be consumed
  // Per-phase device timing (off by default; never during stream capture):
  // one event pair per phase on the stream that runs it, named like the
  // reference's operations ("Dist_s_fusedSynch_allreduce", ...), measured
  // from an origin event on the compute stream.
  bool profiling = false;
  cudaEvent_t prof_origin = nullptr;
  struct Range {
    std::string name;
    cudaEvent_t start, end;
  };
  std::vector<Range> ranges;
  size_t open_range = 0;
  std::vector<void*> registered;   // ncclCommRegister handles (user buffers reduced in place)
  // Staging is deferred: a stage call only records the tensors; the bytes are
  // gathered by ONE multi-tensor pack launch when the bucket is flushed (the
  // tensors must stay alive until then anyway - the flush writes into them).
  std::vector<void*> pend_ptrs;
  std::vector<size_t> pend_sizes;
  size_t pend_off = 0;         // staging-buffer offset of the first pending tensor
  int pend_half = 0;           // pending tensors go to the fp16 staging buffer
};

namespace {

int edge(cudaEvent_t ev, cudaStream_t from, cudaStream_t to) {
  CU(cudaEventRecord(ev, from));
  CU(cudaStreamWaitEvent(to, ev, 0));
  return SGB_OK;
}

cudaStream_t side(const sgb_comm* c, int which) {
  return which == sgb::order::kStreamS ? c->s : (which == sgb::order::kStreamC1 ? c->c1 : c->c2);
}

// Emits the edges of one phase of a planned call (see comm_order.h), in a
// fixed order.  Every edge re-records its event; a wait takes the state of the
// event at the time of the wait, so an event can serve many edges in a row.
int emit(sgb_comm* c, unsigned edges, cudaStream_t compute) {
  using namespace sgb::order;
  if (edges & kComputeToC1) OK(edge(c->ev_compute, compute, c->c1));
  if (edges & kComputeToS) OK(edge(c->ev_compute, compute, c->s));
  if (edges & kC1ToS) OK(edge(c->ev_c1, c->c1, c->s));
  if (edges & kC2DoneToS) CU(cudaStreamWaitEvent(c->s, c->ev_c2_done, 0));
  if (edges & (kSToC1 | kSToC2)) {
    CU(cudaEventRecord(c->ev_s, c->s));
    if (edges & kSToC1) CU(cudaStreamWaitEvent(c->c1, c->ev_s, 0));
    if (edges & kSToC2) CU(cudaStreamWaitEvent(c->c2, c->ev_s, 0));
  }
  if (edges & kMarkC2Done) CU(cudaEventRecord(c->ev_c2_done, c->c2));
  if (edges & kSToCompute) OK(edge(c->ev_s, c->s, compute));
  if (edges & kC1ToCompute) OK(edge(c->ev_c1, c->c1, compute));
  if (edges & kC2ToCompute) OK(edge(c->ev_c2, c->c2, compute));
  return SGB_OK;
}

sgb::order::Step plan_call(sgb_comm* c, int call) {
  sgb::order::Step p = sgb::order::plan(c->order, call);
  c->result_stream = p.result_stream;
  return p;
}

// A named phase on one of the side streams: an NVTX range around the enqueue
// and, while profiling is on, an event pair on that stream.
struct Phase {
  sgb_comm* c;
  cudaStream_t stream;
  bool timed = false;
  size_t slot = 0;
  Phase(sgb_comm* comm, const char* name, int which) : c(comm), stream(side(comm, which)) {
    nvtxRangePushA(name);
    if (!c->profiling) return;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return;
    sgb_comm::Range r;
    r.name = name;
    if (cudaEventCreate(&r.start) != cudaSuccess) return;
    if (cudaEventCreate(&r.end) != cudaSuccess) {
      cudaEventDestroy(r.start);
      return;
    }
    cudaEventRecord(r.start, stream);
    slot = c->ranges.size();
    c->ranges.push_back(r);
    timed = true;
  }
  ~Phase() {
    if (timed) cudaEventRecord(c->ranges[slot].end, stream);
    nvtxRangePop();
  }
};

void drop_ranges(sgb_comm* c) {
  for (auto& r : c->ranges) {
    cudaEventDestroy(r.start);
    if (r.end) cudaEventDestroy(r.end);
  }
  c->ranges.clear();
}

// Packs the deferred tensors into the staging buffer on c1.  The caller has
// emitted compute -> c1 for this call already (every staged gradient was
// produced before this point).
int pack_pending(sgb_comm* c, const char* name) {
  if (c->pend_ptrs.empty()) return SGB_OK;
  Phase ph(c, name, sgb::order::kStreamC1);
  if (c->pend_half)
    OK(sgb_pack_f32_to_f16(c->pend_ptrs.data(), c->pend_sizes.data(), c->pend_ptrs.size(), c->send_h,
                           c->pend_off, c->c1));
  else
    OK(sgb_pack_f32(c->pend_ptrs.data(), c->pend_sizes.data(), c->pend_ptrs.size(), c->send,
                    c->pend_off, c->c1));
  c->pend_ptrs.clear();
  c->pend_sizes.clear();
  return SGB_OK;
}

// A bucket of the other precision is still pending: it is packed now, ordered
// after the compute stream.
int pack_other_kind(sgb_comm* c, cudaStream_t compute, const char* name) {
  OK(emit(c, plan_call(c, sgb::order::kStageCopy).pre, compute));
  return pack_pending(c, name);
}

void defer(sgb_comm* c, void* const* tensors, const size_t* sizes, size_t count, int half) {
  if (c->pend_ptrs.empty()) {
    c->pend_off = c->send_off;
    c->pend_half = half;
  }
  for (size_t i = 0; i < count; ++i) {
    c->pend_ptrs.push_back(tensors[i]);
    c->pend_sizes.push_back(sizes[i]);
  }
}

int half_init(sgb_comm* c) {
  if (c->send_h) return SGB_OK;
  CU(cudaMalloc(&c->send_h, c->max_elems * sizeof(__half)));
  CU(cudaMalloc(&c->recv_h, c->max_elems * sizeof(__half)));
  CU(cudaMalloc(&c->dsend_h, c->max_elems * sizeof(__half)));
  CU(cudaMalloc(&c->drecv_h, c->max_elems * sizeof(__half)));
  return SGB_OK;
}

int sparse_init(sgb_comm* c) {
  if (c->pay_send) return SGB_OK;
  const size_t n = c->max_elems;
  CU(cudaMalloc(&c->pay_send, 2 * n * sizeof(int)));
  CU(cudaMalloc(&c->pay_recv, 2 * n * sizeof(int) * static_cast<size_t>(c->world)));
  c->ws_bytes = sgb_sparse_workspace_bytes(n);
  CU(cudaMalloc(&c->ws, c->ws_bytes));
  CU(cudaMalloc(&c->nnz_dev, sizeof(int) * (c->world + 1)));
  CU(cudaMallocHost(&c->nnz_host, sizeof(int) * c->world));
  CU(cudaMalloc(&c->dropped_dev, sizeof(unsigned long long)));
  CU(cudaMemset(c->dropped_dev, 0, sizeof(unsigned long long)));
  return SGB_OK;
}

size_t total_of(const size_t* sizes, size_t count) {
  size_t t = 0;
  for (size_t i = 0; i < count; ++i) t += sizes[i];
  return t;
}

int check_list(void* const* tensors, const size_t* sizes, size_t count) {
  if (count == 0) return SGB_ERR_SIZE;  // the reference CHECKs t.size() > 0
  if (!tensors || !sizes) return SGB_ERR_NULL;
  for (size_t i = 0; i < count; ++i)
    if (sizes[i] && !tensors[i]) return SGB_ERR_NULL;
  return SGB_OK;
}

}  // namespace

extern "C" {

int sgb_last_nccl_error(void) { return g_last_nccl_error.load(); }

int sgb_comm_unique_id_bytes(void) { return static_cast<int>(sizeof(ncclUniqueId)); }

int sgb_comm_get_unique_id(void* id_out) {
  if (!id_out) return SGB_ERR_NULL;
  ncclUniqueId id;
  NC(ncclGetUniqueId(&id));
  std::memcpy(id_out, &id, sizeof(id));
  return SGB_OK;
}

int sgb_comm_create(sgb_comm** out, int rank, int world, const void* unique_id, size_t max_elems) {
  return sgb_comm_create_ex(out, rank, world, unique_id, max_elems, 0, 0);
}

int sgb_comm_register(sgb_comm* c, void* buffer, size_t bytes) {
  if (!c || !buffer) return SGB_ERR_NULL;
  if (bytes == 0) return SGB_ERR_SIZE;
  void* handle = nullptr;
  NC(ncclCommRegister(c->nccl, buffer, bytes, &handle));
  c->registered.push_back(handle);
  return SGB_OK;
}

int sgb_comm_create_ex(sgb_comm** out, int rank, int world, const void* unique_id, size_t max_elems,
                       int min_ctas, int max_ctas) {
  if (!out || !unique_id) return SGB_ERR_NULL;
  if (world < 1 || rank < 0 || rank >= world || max_elems == 0) return SGB_ERR_SIZE;
  if (max_elems > 0x7fffffffu) return SGB_ERR_SIZE;  // collective counts and 1-based indices are int32
  sgb_comm* c = new (std::nothrow) sgb_comm();
  if (!c) return SGB_ERR_STATE;
  c->rank = rank;
  c->world = world;
  c->max_elems = max_elems;
  *out = c;  // handed out early so a failed create can still be destroyed
  CU(cudaGetDevice(&c->device));
  ncclUniqueId id;
  std::memcpy(&id, unique_id, sizeof(id));
  if (min_ctas > 0 || max_ctas > 0) {
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    if (min_ctas > 0) cfg.minCTAs = min_ctas;
    if (max_ctas > 0) cfg.maxCTAs = max_ctas;
    NC(ncclCommInitRankConfig(&c->nccl, world, id, rank, &cfg));
  } else {
    NC(ncclCommInitRank(&c->nccl, world, id, rank));
  }
  CU(cudaMalloc(&c->send, max_elems * sizeof(float)));
  CU(cudaMalloc(&c->recv, max_elems * sizeof(float)));
  // Highest priority: the collectives and their small pack / unpack kernels
  // should start as soon as their inputs exist instead of queueing behind the
  // large backward kernels of the compute stream.
  int prio_lo = 0, prio_hi = 0;
  CU(cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi));
  CU(cudaStreamCreateWithPriority(&c->s, cudaStreamNonBlocking, prio_hi));
  CU(cudaStreamCreateWithPriority(&c->c1, cudaStreamNonBlocking, prio_hi));
  CU(cudaStreamCreateWithPriority(&c->c2, cudaStreamNonBlocking, prio_hi));
  cudaEvent_t* evs[] = {&c->ev_compute, &c->ev_c1, &c->ev_s, &c->ev_c2, &c->ev_c2_done};
  for (cudaEvent_t* e : evs) CU(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
  CU(cudaEventCreateWithFlags(&c->ev_host, cudaEventDisableTiming | cudaEventBlockingSync));
  return SGB_OK;
}

int sgb_comm_destroy(sgb_comm* c) {
  if (!c) return SGB_OK;
  if (c->s) cudaStreamSynchronize(c->s);
  if (c->c1) cudaStreamSynchronize(c->c1);
  if (c->c2) cudaStreamSynchronize(c->c2);
  if (c->nccl) {
    for (void* h : c->registered) ncclCommDeregister(c->nccl, h);
    ncclCommDestroy(c->nccl);
  }
  void* bufs[] = {c->send, c->recv, c->send_h, c->recv_h, c->dsend_h, c->drecv_h, c->sum, c->pay_send,
                  c->pay_recv, c->ws, c->nnz_dev};
  for (void* b : bufs)
    if (b) cudaFree(b);
  if (c->nnz_host) cudaFreeHost(c->nnz_host);
  if (c->dropped_dev) cudaFree(c->dropped_dev);
  drop_ranges(c);
  cudaEvent_t evs[] = {c->ev_compute, c->ev_c1, c->ev_s, c->ev_c2, c->ev_c2_done, c->ev_host, c->prof_origin};
  for (cudaEvent_t e : evs)
    if (e) cudaEventDestroy(e);
  cudaStream_t ss[] = {c->s, c->c1, c->c2};
  for (cudaStream_t st : ss)
    if (st && c->own_streams) cudaStreamDestroy(st);
  delete c;
  return SGB_OK;
}

int sgb_comm_use_streams(sgb_comm* c, void* s, void* c1, void* c2) {
  if (!c || !s || !c1 || !c2) return SGB_ERR_NULL;
  if (s == c1 || s == c2 || c1 == c2) return SGB_ERR_UNSUPPORTED;
  if (c->order.dirty_s || c->order.dirty_c1 || c->order.dirty_c2 || !c->pend_ptrs.empty()) return SGB_ERR_STATE;
  if (c->own_streams) {
    cudaStream_t ss[] = {c->s, c->c1, c->c2};
    for (cudaStream_t st : ss)
      if (st) {
        CU(cudaStreamSynchronize(st));
        CU(cudaStreamDestroy(st));
      }
  }
  c->s = sgb::as_stream(s);
  c->c1 = sgb::as_stream(c1);
  c->c2 = sgb::as_stream(c2);
  c->own_streams = false;
  return SGB_OK;
}

int sgb_comm_rank(const sgb_comm* c) { return c ? c->rank : -1; }
int sgb_comm_world_size(const sgb_comm* c) { return c ? c->world : -1; }
size_t sgb_comm_staged_elems(const sgb_comm* c) { return c ? c->send_off : 0; }

int sgb_comm_set_topk_mode(sgb_comm* c, int mode) {
  if (!c) return SGB_ERR_NULL;
  if (mode != 0 && mode != 1) return SGB_ERR_UNSUPPORTED;
  c->topk_mode = mode;
  return SGB_OK;
}

/* The three side streams, for callers that profile or order against them:
 * which = 0 (s, NCCL), 1 (c1), 2 (c2). */
void* sgb_comm_stream(const sgb_comm* c, int which) {
  if (!c) return nullptr;
  return which == 0 ? c->s : (which == 1 ? c->c1 : (which == 2 ? c->c2 : nullptr));
}

int sgb_comm_wait(sgb_comm* c, void* compute_stream) {
  if (!c) return SGB_ERR_NULL;
  return emit(c, plan_call(c, sgb::order::kWait).before, sgb::as_stream(compute_stream));
}

void* sgb_comm_result_stream(const sgb_comm* c) { return c ? side(c, c->result_stream) : nullptr; }

int sgb_comm_order_plan(unsigned char* state, int call, unsigned* edges, int* result_stream) {
  if (!state || !edges) return SGB_ERR_NULL;
  if (call < sgb::order::kSynch || call > sgb::order::kWait) return SGB_ERR_UNSUPPORTED;
  sgb::order::State st;
  st.dirty_s = state[0];
  st.dirty_c1 = state[1];
  st.dirty_c2 = state[2];
  st.c2_reads_recv = state[3];
  const sgb::order::Step p = sgb::order::plan(st, call);
  state[0] = st.dirty_s;
  state[1] = st.dirty_c1;
  state[2] = st.dirty_c2;
  state[3] = st.c2_reads_recv;
  edges[0] = p.pre;
  edges[1] = p.before;
  edges[2] = p.after;
  edges[3] = p.post;
  if (result_stream) *result_stream = p.result_stream;
  return SGB_OK;
}

int sgb_comm_profile_begin(sgb_comm* c, void* compute_stream) {
  if (!c) return SGB_ERR_NULL;
  drop_ranges(c);
  if (!c->prof_origin) CU(cudaEventCreate(&c->prof_origin));
  CU(cudaEventRecord(c->prof_origin, sgb::as_stream(compute_stream)));
  c->profiling = true;
  return SGB_OK;
}

int sgb_comm_profile_range(sgb_comm* c, const char* name, int which, int begin) {
  if (!c || !name) return SGB_ERR_NULL;
  if (which < 0 || which > 2) return SGB_ERR_UNSUPPORTED;
  if (!c->profiling) return SGB_OK;
  if (begin) {
    sgb_comm::Range r;
    r.name = name;
    CU(cudaEventCreate(&r.start));
    CU(cudaEventCreate(&r.end));
    CU(cudaEventRecord(r.start, side(c, which)));
    c->open_range = c->ranges.size();
    c->ranges.push_back(r);
  } else if (c->open_range < c->ranges.size()) {
    CU(cudaEventRecord(c->ranges[c->open_range].end, side(c, which)));
  }
  return SGB_OK;
}

int sgb_comm_profile_mark(sgb_comm* c, const char* name, void* stream) {
  if (!c || !name) return SGB_ERR_NULL;
  if (!c->profiling) return SGB_OK;
  sgb_comm::Range r;
  r.name = name;
  CU(cudaEventCreate(&r.start));
  CU(cudaEventRecord(r.start, sgb::as_stream(stream)));
  r.end = nullptr;   // a mark has no extent
  c->ranges.push_back(r);
  return SGB_OK;
}

int sgb_comm_profile_end(sgb_comm* c, char* names, size_t name_stride, float* start_ms, float* end_ms,
                         size_t capacity, size_t* count) {
  if (!c || !count) return SGB_ERR_NULL;
  c->profiling = false;
  CU(cudaDeviceSynchronize());
  *count = c->ranges.size();
  for (size_t i = 0; i < c->ranges.size() && i < capacity; ++i) {
    const sgb_comm::Range& r = c->ranges[i];
    if (names && name_stride) {
      std::strncpy(names + i * name_stride, r.name.c_str(), name_stride - 1);
      names[i * name_stride + name_stride - 1] = 0;
    }
    if (start_ms) CU(cudaEventElapsedTime(start_ms + i, c->prof_origin, r.start));
    if (end_ms) CU(cudaEventElapsedTime(end_ms + i, c->prof_origin, r.end ? r.end : r.start));
  }
  drop_ranges(c);
  return SGB_OK;
}

int sgb_comm_synch(sgb_comm* c, void* data, size_t n, int is_half, void* compute_stream) {
  if (!c) return SGB_ERR_NULL;
  if (n == 0) return SGB_OK;
  if (!data) return SGB_ERR_NULL;
  if (n > 0x7fffffffu) return SGB_ERR_SIZE;
  const sgb::order::Step p = plan_call(c, sgb::order::kSynch);
  OK(emit(c, p.before, sgb::as_stream(compute_stream)));
  {
    Phase ph(c, "Dist_s_synch_allreduce", sgb::order::kStreamS);
    NC(ncclAllReduce(data, data, n, is_half ? ncclHalf : ncclFloat, ncclSum, c->nccl, c->s));
  }
  return emit(c, p.after, nullptr);
}

int sgb_comm_fused_synch(sgb_comm* c, void* const* tensors, const size_t* sizes, size_t count,
                         int is_half, int send, void* compute_stream) {
  if (!c) return SGB_ERR_NULL;
  OK(check_list(tensors, sizes, count));
  cudaStream_t compute = sgb::as_stream(compute_stream);
  const size_t esz = is_half ? sizeof(__half) : sizeof(float);
  if (!send) {
    const size_t total = total_of(sizes, count);
    if (c->send_off + total > c->max_elems) return SGB_ERR_CAPACITY;
    if (!is_half) {
      if (!c->pend_ptrs.empty() && c->pend_half)
        OK(pack_other_kind(c, compute, "Dist_c1_fusedSynchHalf_filling"));
      defer(c, tensors, sizes, count, 0);
    } else {
      OK(emit(c, plan_call(c, sgb::order::kStageCopy).pre, compute));
      Phase ph(c, "Dist_c1_fusedSynch_filling", sgb::order::kStreamC1);
      size_t off = c->send_off;
      for (size_t i = 0; i < count; ++i) {
        CU(cudaMemcpyAsync(reinterpret_cast<char*>(c->send) + off * esz, tensors[i],
                           sizes[i] * esz, cudaMemcpyDeviceToDevice, c->c1));
        off += sizes[i];
      }
    }
    c->send_off += total;
    return SGB_OK;
  }
  // flush: everything staged so far is reduced; `tensors` receive the result
  const size_t total = total_of(sizes, count);
  if (total > c->max_elems) return SGB_ERR_CAPACITY;
  // Gradients that already sit back to back in memory (a gradient arena) need
  // neither the pack nor the unpack pass: the bucket is reduced in place, on s,
  // ordered directly after the compute stream that produced it.
  if (!is_half && !c->pend_half && c->pend_off == 0 && c->pend_ptrs.size() == count &&
      c->send_off == total) {
    bool in_place = true;
    for (size_t i = 0; i < count && in_place; ++i) {
      in_place = c->pend_ptrs[i] == tensors[i] && c->pend_sizes[i] == sizes[i] &&
                 (i + 1 == count ||
                  static_cast<char*>(tensors[i]) + sizes[i] * sizeof(float) == tensors[i + 1]);
    }
    if (in_place) {
      c->pend_ptrs.clear();
      c->pend_sizes.clear();
      c->send_off = 0;
      const sgb::order::Step p = plan_call(c, sgb::order::kFlushInPlace);
      OK(emit(c, p.before, compute));
      {
        Phase ph(c, "Dist_s_fusedSynch_allreduce", sgb::order::kStreamS);
        NC(ncclAllReduce(tensors[0], tensors[0], total, ncclFloat, ncclSum, c->nccl, c->s));
      }
      return emit(c, p.after, nullptr);
    }
  }
  const sgb::order::Step p = plan_call(c, sgb::order::kFlushPacked);
  OK(emit(c, p.pre, compute));
  OK(pack_pending(c, "Dist_c1_fusedSynch_filling"));
  OK(emit(c, p.before, compute));
  if (c->send_off) {
    Phase ph(c, "Dist_s_fusedSynch_allreduce", sgb::order::kStreamS);
    NC(ncclAllReduce(c->send, c->recv, c->send_off, is_half ? ncclHalf : ncclFloat, ncclSum,
                     c->nccl, c->s));
  }
  c->send_off = 0;
  OK(emit(c, p.after, nullptr));
  Phase ph(c, "Dist_c1_fusedSynch_copyBackToTensor", sgb::order::kStreamC1);
  if (!is_half) {
    OK(sgb_unpack_f32(c->recv, 0, tensors, sizes, count, 1.0f, c->c1));
  } else {
    size_t off = 0;
    for (size_t i = 0; i < count; ++i) {
      CU(cudaMemcpyAsync(tensors[i], reinterpret_cast<char*>(c->recv) + off * esz, sizes[i] * esz,
                         cudaMemcpyDeviceToDevice, c->c1));
      off += sizes[i];
    }
  }
  return SGB_OK;
}

int sgb_comm_synch_half(sgb_comm* c, float* data, size_t n, void* compute_stream) {
  if (!c) return SGB_ERR_NULL;
  if (n == 0) return SGB_OK;
  if (!data) return SGB_ERR_NULL;
  if (n > c->max_elems) return SGB_ERR_CAPACITY;
  OK(half_init(c));
  cudaStream_t compute = sgb::as_stream(compute_stream);
  const sgb::order::Step p = plan_call(c, sgb::order::kSynchHalf);
  OK(emit(c, p.pre, compute));
  {
    Phase ph(c, "Dist_c1_synchHalf_float2half", sgb::order::kStreamC1);
    OK(sgb_cast_f32_f16(data, c->dsend_h, n, c->c1));
  }
  OK(emit(c, p.before, compute));
  {
    Phase ph(c, "Dist_s_synchHalf_allreduce", sgb::order::kStreamS);
    NC(ncclAllReduce(c->dsend_h, c->drecv_h, n, ncclHalf, ncclSum, c->nccl, c->s));
  }
  OK(emit(c, p.after, nullptr));
  {
    Phase ph(c, "Dist_c2_synchHalf_half2float", sgb::order::kStreamC2);
    OK(sgb_cast_f16_f32(c->drecv_h, data, n, c->c2));
  }
  return emit(c, p.post, nullptr);
}

int sgb_comm_fused_synch_half(sgb_comm* c, void* const* tensors, const size_t* sizes,
                              size_t count, int send, void* compute_stream) {
  if (!c) return SGB_ERR_NULL;
  OK(check_list(tensors, sizes, count));
  OK(half_init(c));
  cudaStream_t compute = sgb::as_stream(compute_stream);
  const size_t total = total_of(sizes, count);
  if (!send) {
    if (c->send_off + total > c->max_elems) return SGB_ERR_CAPACITY;
    // copy + float2half of the reference collapse into one pack-and-cast pass at flush time
    if (!c->pend_ptrs.empty() && !c->pend_half)
      OK(pack_other_kind(c, compute, "Dist_c1_fusedSynch_filling"));
    defer(c, tensors, sizes, count, 1);
    c->send_off += total;
    return SGB_OK;
  }
  if (total > c->max_elems) return SGB_ERR_CAPACITY;
  const sgb::order::Step p = plan_call(c, sgb::order::kFlushHalf);
  OK(emit(c, p.pre, compute));
  OK(pack_pending(c, "Dist_c1_fusedSynchHalf_float2half"));
  OK(emit(c, p.before, compute));
  if (c->send_off) {
    Phase ph(c, "Dist_s_fusedSynchHalf_allreduce", sgb::order::kStreamS);
    NC(ncclAllReduce(c->send_h, c->recv_h, c->send_off, ncclHalf, ncclSum, c->nccl, c->s));
  }
  c->send_off = 0;
  OK(emit(c, p.after, nullptr));
  {
    Phase ph(c, "Dist_c2_fusedSynchHalf_half2floatcopy", sgb::order::kStreamC2);
    OK(sgb_unpack_f16_to_f32(c->recv_h, 0, tensors, sizes, count, 1.0f, c->c2));
  }
  return emit(c, p.post, nullptr);
}

// capacity == 0: the reference's exchange (the payload is as long as the
// largest count, which the host reads back).  capacity > 0 (threshold mode):
// every rank sends exactly `capacity` slots, no host round trip.
static int sparsify(sgb_comm* c, void* const* tensors, const size_t* sizes, size_t count,
                    float* accumulation, float spars, int topk, size_t capacity, void* compute_stream) {
  if (!c) return SGB_ERR_NULL;
  OK(check_list(tensors, sizes, count));
  const size_t n = total_of(sizes, count);
  if (n > c->max_elems) return SGB_ERR_CAPACITY;
  if (capacity > c->max_elems) return SGB_ERR_CAPACITY;
  if (n == 0) return SGB_OK;
  OK(sparse_init(c));
  const int W = c->world;
  const char* op_name = count > 1 ? "Dist_c1c2_fusedSparsification" : "Dist_c1c2_sparsification";
  const sgb::order::Step p = plan_call(c, sgb::order::kSparse);
  OK(emit(c, p.pre, sgb::as_stream(compute_stream)));
  // One tensor, or tensors that lie back to back in memory (a gradient arena),
  // are selected from and scattered into IN PLACE: no copy into the send
  // buffer and none back (16 B/element saved).  The selection has finished
  // reading the gradient before the dense result is written: c1 -> s -> c2.
  bool in_place = sgb::aligned16(tensors[0]);
  for (size_t i = 1; i < count && in_place; ++i)
    in_place = static_cast<const float*>(tensors[i]) == static_cast<const float*>(tensors[i - 1]) + sizes[i - 1];
  float* grad = in_place ? static_cast<float*>(tensors[0]) : c->send;
  float* dense = in_place ? static_cast<float*>(tensors[0]) : c->recv;

  size_t nnz_max = 0;
  auto select = [&]() -> int {
  Phase ph(c, op_name, sgb::order::kStreamC1);
  if (!in_place) OK(sgb_pack_f32(tensors, sizes, count, c->send, 0, c->c1));
  if (!topk && capacity) {
    OK(sgb::sparse_threshold_count(grad, accumulation, n, spars, c->nnz_dev, c->ws,
                                   c->ws_bytes, c->c1));
    // the counts travel on the device only; receivers clamp them to the capacity
    NC(ncclAllGather(c->nnz_dev, c->nnz_dev + 1, 1, ncclInt, c->nccl, c->c1));
    OK(sgb::sparse_threshold_write_bounded(grad, accumulation, n, spars, c->pay_send, capacity, c->dropped_dev,
                                           c->ws, c->c1));
    nnz_max = capacity;
  } else if (!topk) {
    OK(sgb::sparse_threshold_count(grad, accumulation, n, spars, c->nnz_dev, c->ws,
                                   c->ws_bytes, c->c1));
    NC(ncclAllGather(c->nnz_dev, c->nnz_dev + 1, 1, ncclInt, c->nccl, c->c1));
    CU(cudaMemcpyAsync(c->nnz_host, c->nnz_dev + 1, sizeof(int) * W, cudaMemcpyDeviceToHost, c->c1));
    CU(cudaEventRecord(c->ev_host, c->c1));
    // the compaction runs while the host waits for the counts
    OK(sgb::sparse_threshold_write_packed(grad, accumulation, n, spars, c->pay_send, c->ws, c->c1));
    CU(cudaEventSynchronize(c->ev_host));
    for (int r = 0; r < W; ++r) {
      if (c->nnz_host[r] < 0 || static_cast<size_t>(c->nnz_host[r]) > n) return SGB_ERR_STATE;
      if (static_cast<size_t>(c->nnz_host[r]) > nnz_max) nnz_max = c->nnz_host[r];
    }
  } else {
    nnz_max = static_cast<size_t>(sgb_topk_count(spars, n));
    for (int r = 0; r < W; ++r) c->nnz_host[r] = static_cast<int>(nnz_max);
    if (nnz_max)
      OK(sgb_sparse_topk_f32(grad, accumulation, nullptr, n, nnz_max, c->topk_mode, c->pay_send,
                             reinterpret_cast<float*>(c->pay_send) + nnz_max, c->ws, c->ws_bytes,
                             c->c1));
  }
  return SGB_OK;
  };
  OK(select());

  OK(emit(c, p.before, sgb::as_stream(compute_stream)));
  if (nnz_max) {
    Phase ph(c, "Dist_s_sparsification_allgather", sgb::order::kStreamS);
    NC(ncclAllGather(c->pay_send, c->pay_recv, 2 * nnz_max, ncclFloat, c->nccl, c->s));
  }
  OK(emit(c, p.after, nullptr));
  auto scatter = [&]() -> int {
  Phase ph(c, op_name, sgb::order::kStreamC2);
  CU(cudaMemsetAsync(dense, 0, n * sizeof(float), c->c2));
  for (int r = 0; r < W && nnz_max; ++r) {  // ranks in ascending order, as the reference
    const int* seg = c->pay_recv + static_cast<size_t>(r) * 2 * nnz_max;
    if (capacity) {                                   // fixed layout; the rank's count is read on the device
      OK(sgb_scatter_add_f32(seg, reinterpret_cast<const float*>(seg) + capacity, capacity, c->nnz_dev + 1 + r,
                             dense, n, c->c2));
      continue;
    }
    const size_t cnt = static_cast<size_t>(c->nnz_host[r]);
    OK(sgb_scatter_add_f32(seg, reinterpret_cast<const float*>(seg) + cnt, cnt, nullptr, dense,
                           n, c->c2));
  }
  if (!in_place) OK(sgb_unpack_f32(c->recv, 0, tensors, sizes, count, 1.0f, c->c2));
  return SGB_OK;
  };
  OK(scatter());
  return emit(c, p.post, nullptr);
}

int sgb_comm_sparsification(sgb_comm* c, void* const* tensors, const size_t* sizes, size_t count,
                            float* accumulation, float spars, int topk, void* compute_stream) {
  return sparsify(c, tensors, sizes, count, accumulation, spars, topk, 0, compute_stream);
}

int sgb_comm_sparsification_bounded(sgb_comm* c, void* const* tensors, const size_t* sizes, size_t count,
                                    float* accumulation, float threshold, size_t capacity,
                                    void* compute_stream) {
  if (capacity == 0) return SGB_ERR_SIZE;
  return sparsify(c, tensors, sizes, count, accumulation, threshold, 0, capacity, compute_stream);
}

int sgb_comm_sparse_dropped(sgb_comm* c, unsigned long long* dropped) {
  if (!c || !dropped) return SGB_ERR_NULL;
  *dropped = 0;
  if (!c->dropped_dev) return SGB_OK;               // no sparse call yet
  // on the stream that runs the selection, so that every call issued so far is counted
  CU(cudaMemcpyAsync(dropped, c->dropped_dev, sizeof(unsigned long long), cudaMemcpyDeviceToHost, c->c1));
  CU(cudaStreamSynchronize(c->c1));
  return SGB_OK;
}

}  // extern "C"
