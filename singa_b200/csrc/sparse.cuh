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

}  // namespace sgb
