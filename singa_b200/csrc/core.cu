// Library-wide state: status strings, error bookkeeping, device properties.
#include <atomic>

#include "common.cuh"

namespace sgb {
namespace {
std::atomic<int> g_last_cuda_error{0};
constexpr int kMaxDevices = 64;
std::atomic<int> g_sm_count[kMaxDevices];
std::atomic<int> g_options[SGB_OPT_COUNT_];
struct OptionDefaults {
  OptionDefaults() { g_options[SGB_OPT_OVERLAP_LAUNCHES].store(1); }
} g_option_defaults;
}  // namespace

int option(int which) {
  return which > 0 && which < SGB_OPT_COUNT_ ? g_options[which].load(std::memory_order_relaxed) : 0;
}

int note_cuda_error(cudaError_t e) {
  g_last_cuda_error.store(static_cast<int>(e));
  return SGB_ERR_CUDA;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int v = g_sm_count[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
    v = 148;
  g_sm_count[dev].store(v, std::memory_order_relaxed);
  return v;
}
}  // namespace sgb

extern "C" {

const char* sgb_status_string(int status) {
  switch (status) {
    case SGB_OK: return "ok";
    case SGB_ERR_NULL: return "required pointer is NULL";
    case SGB_ERR_SIZE: return "inconsistent or out-of-range size";
    case SGB_ERR_CUDA: return "CUDA runtime error (see sgb_last_cuda_error)";
    case SGB_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
    case SGB_ERR_NCCL: return "NCCL error (see sgb_last_nccl_error)";
    case SGB_ERR_UNSUPPORTED: return "unsupported op, dtype or mode";
    case SGB_ERR_STATE: return "call not valid in this state";
    case SGB_ERR_CAPACITY: return "does not fit the communicator's buffers";
    case SGB_ERR_LIMIT: return "size exceeds the built-in scratch of this entry point (limit stated in sgb.h)";
    default: return "unknown status";
  }
}

int sgb_last_cuda_error(void) { return sgb::g_last_cuda_error.load(); }

int sgb_version(void) { return 110; }

int sgb_set_option(int option, int value) {
  if (option <= 0 || option >= SGB_OPT_COUNT_) return SGB_ERR_UNSUPPORTED;
  sgb::g_options[option].store(value);
  return SGB_OK;
}

int sgb_get_option(int option) { return sgb::option(option); }

}  // extern "C"
