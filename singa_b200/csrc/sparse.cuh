// Internal two-phase interface of the threshold sparsifier, used by the
// communicator so that the payload length can travel to the host while the
// compaction kernel is already running.
#pragma once
#include "common.cuh"

namespace sgb {

// Phase 1: per-tile counts + scan; the payload length lands in *nnz_dev.
int sparse_threshold_count(const float* g, float* acc, size_t n, float thr, int* nnz_dev,
                           void* ws, size_t ws_bytes, cudaStream_t s);

// Phase 2: residual update and packed payload [idx(nnz) | val(nnz)] written to
// `payload` (int32 view), using the offsets left in `ws` by phase 1.
int sparse_threshold_write_packed(const float* g, float* acc, size_t n, float thr, int* payload,
                                  void* ws, cudaStream_t s);

// Phase 2, capacity-bounded: payload [idx(cap) | val(cap)]; selected entries
// beyond the first `cap` (index order) stay in the residual and are counted in
// *dropped_dev (a device counter the caller owns).
int sparse_threshold_write_bounded(const float* g, float* acc, size_t n, float thr, int* payload, size_t cap,
                                   unsigned long long* dropped_dev, void* ws, cudaStream_t s);

}  // namespace sgb
