// Stand-in for NVIDIA's cnmem library (an external, un-vendored dependency of
// apache/singa: include/singa/core/memory.h:29, src/core/memory/memory.cc) for
// builds of the reference's CUDA device classes in the checker.  The seven
// entry points the reference calls are provided over cudaMalloc with a
// size-keyed free list: a freed block is handed to the next request of the
// same size without a cudaFree, which keeps the property the reference's graph
// scheduler relies on (memory released on the host while kernels are queued is
// only reused by later work of the same stream).  TEST INFRASTRUCTURE ONLY.
#ifndef SGB_REF_CNMEM_H_
#define SGB_REF_CNMEM_H_
#include <cuda_runtime.h>

#include <cstddef>
#include <map>
#include <mutex>
#include <vector>

typedef enum {
  CNMEM_STATUS_SUCCESS = 0,
  CNMEM_STATUS_CUDA_ERROR,
  CNMEM_STATUS_INVALID_ARGUMENT,
  CNMEM_STATUS_NOT_INITIALIZED,
  CNMEM_STATUS_OUT_OF_MEMORY,
  CNMEM_STATUS_UNKNOWN_ERROR
} cnmemStatus_t;

typedef enum { CNMEM_FLAGS_DEFAULT = 0, CNMEM_FLAGS_CANNOT_GROW = 1, CNMEM_FLAGS_CANNOT_STEAL = 2 } cnmemManagerFlags_t;

typedef struct cnmemDevice_t_ {
  int device;
  size_t size;
  int numStreams;
  cudaStream_t* streams;
  size_t* streamSizes;
} cnmemDevice_t;

namespace sgb_cnmem {
struct Pool {
  std::mutex mu;
  std::map<size_t, std::vector<void*>> free_blocks;   // by rounded size
  std::map<void*, size_t> live;                       // every block ever handed out -> rounded size
};
// Never destroyed: the device that owns the memory pool is itself a static
// (Platform::UsedDevice) and finalises the pool from its destructor at process
// exit, possibly after a function-local static here would already be gone.
inline Pool& pool() {
  static Pool* p = new Pool;
  return *p;
}
inline size_t rounded(size_t n) { return (n + 511) & ~static_cast<size_t>(511); }
}  // namespace sgb_cnmem

inline const char* cnmemGetErrorString(cnmemStatus_t s) {
  switch (s) {
    case CNMEM_STATUS_SUCCESS: return "CNMEM_STATUS_SUCCESS";
    case CNMEM_STATUS_CUDA_ERROR: return "CNMEM_STATUS_CUDA_ERROR";
    case CNMEM_STATUS_INVALID_ARGUMENT: return "CNMEM_STATUS_INVALID_ARGUMENT";
    case CNMEM_STATUS_NOT_INITIALIZED: return "CNMEM_STATUS_NOT_INITIALIZED";
    case CNMEM_STATUS_OUT_OF_MEMORY: return "CNMEM_STATUS_OUT_OF_MEMORY";
    default: return "CNMEM_STATUS_UNKNOWN_ERROR";
  }
}

inline cnmemStatus_t cnmemInit(int, const cnmemDevice_t*, unsigned) { return CNMEM_STATUS_SUCCESS; }

inline cnmemStatus_t cnmemFinalize() {
  sgb_cnmem::Pool& p = sgb_cnmem::pool();
  std::lock_guard<std::mutex> lock(p.mu);
  for (auto& kv : p.free_blocks)
    for (void* b : kv.second) {
      cudaFree(b);
      p.live.erase(b);
    }
  p.free_blocks.clear();
  return CNMEM_STATUS_SUCCESS;
}

inline cnmemStatus_t cnmemMalloc(void** ptr, size_t size, cudaStream_t) {
  if (!ptr) return CNMEM_STATUS_INVALID_ARGUMENT;
  sgb_cnmem::Pool& p = sgb_cnmem::pool();
  const size_t r = sgb_cnmem::rounded(size ? size : 1);
  std::lock_guard<std::mutex> lock(p.mu);
  auto it = p.free_blocks.find(r);
  if (it != p.free_blocks.end() && !it->second.empty()) {
    *ptr = it->second.back();
    it->second.pop_back();
    return CNMEM_STATUS_SUCCESS;
  }
  if (cudaMalloc(ptr, r) != cudaSuccess) return CNMEM_STATUS_OUT_OF_MEMORY;
  p.live[*ptr] = r;
  return CNMEM_STATUS_SUCCESS;
}

inline cnmemStatus_t cnmemFree(void* ptr, cudaStream_t) {
  if (!ptr) return CNMEM_STATUS_SUCCESS;
  sgb_cnmem::Pool& p = sgb_cnmem::pool();
  std::lock_guard<std::mutex> lock(p.mu);
  auto it = p.live.find(ptr);
  if (it == p.live.end()) return CNMEM_STATUS_INVALID_ARGUMENT;
  p.free_blocks[it->second].push_back(ptr);
  return CNMEM_STATUS_SUCCESS;
}

inline cnmemStatus_t cnmemMemGetInfo(size_t* free_bytes, size_t* total_bytes, cudaStream_t) {
  return cudaMemGetInfo(free_bytes, total_bytes) == cudaSuccess ? CNMEM_STATUS_SUCCESS : CNMEM_STATUS_CUDA_ERROR;
}
#endif  // SGB_REF_CNMEM_H_
