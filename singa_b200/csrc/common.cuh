// Shared device/host helpers for the sm_100a kernels behind the C ABI.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "sgb.h"

namespace sgb {

// Number of SMs of the current device (148 on B200), cached per device.
int sm_count();

// Records a CUDA runtime error so sgb_last_cuda_error() can report it.
int note_cuda_error(cudaError_t e);

// Returns SGB_OK or SGB_ERR_CUDA after a kernel launch (launch errors only;
// nothing here synchronises).
inline int launch_status() {
  cudaError_t e = cudaPeekAtLastError();
  return e == cudaSuccess ? SGB_OK : note_cuda_error(cudaGetLastError());
}

inline bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// Library-wide switches (sgb_set_option); read on the host at launch time.
int option(int which);

// Launch with optional attributes: a thread-block cluster of `cluster` CTAs
// along x (0 = none) and, when SGB_OPT_OVERLAP_LAUNCHES is on and the kernel
// is `dependent_aware`, programmatic stream serialisation: the grid may be
// scheduled while the previous kernel of the stream drains, and the kernel
// itself waits (dependency_wait) before it touches global memory.  Only
// kernels that contain that wait may pass dependent_aware = true.
template <typename... KArgs, typename... Args>
inline int launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                     int cluster, bool dependent_aware, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster > 0) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (dependent_aware && option(SGB_OPT_OVERLAP_LAUNCHES)) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return note_cuda_error(e);
  return launch_status();
}

// Grid for a grid-stride kernel: enough CTAs for the work, capped at
// ctas_per_sm resident CTAs on every SM so the grid is a multiple of the SM
// count when the problem is large.
inline unsigned capped_grid(size_t work_items, size_t per_cta, int ctas_per_sm) {
  size_t need = ceil_div(work_items, per_cta);
  size_t cap = static_cast<size_t>(sm_count()) * ctas_per_sm;
  if (need < 1) need = 1;
  return static_cast<unsigned>(need < cap ? need : cap);
}

// ---------------------------------------------------------------- device side
// Programmatic dependent launch.  dependency_wait: returns once every kernel
// this grid depends on has completed and its writes are visible (a no-op for
// a grid launched without the attribute).  It must precede the first access
// to global memory.  release_dependents: this CTA no longer needs the SM's
// free resources for CTAs of its own grid; once every CTA of the grid has
// said so (or exited), the next kernel of the stream may be scheduled.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed combination order (deterministic run to run).
// smem must hold 32 floats.  Result valid in every thread.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protects smem reuse across consecutive calls
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  float r = lane < nwarp ? smem[lane] : 0.0f;
  r = warp_sum(r);
  return r;
}

// 128-bit global accesses.  "Streaming" forms mark the line evict-first: the
// gradient tensors on this path are touched once per step.
__device__ __forceinline__ uint4 ld128(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ uint4 ld128_stream(const void* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st128(void* p, uint4 v) {
  *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ void st128_stream(void* p, uint4 v) {
  __stcs(reinterpret_cast<uint4*>(p), v);
}

union Vec4f {
  uint4 u;
  float f[4];
  int i[4];
};
union Vec8h {
  uint4 u;
  __half h[8];
  __half2 h2[4];
};

}  // namespace sgb
