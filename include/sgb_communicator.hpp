/* C++ host-side mirror of singa::Communicator (include/singa/io/communicator.h:
 * 69-95: NcclIdHolder and the public interface of Communicator) over the C ABI
 * of sgb.h.  Header only; needs no CUDA or NCCL header.
 *
 * Same method names, argument meaning and error behaviour as the reference:
 * a failed call prints the reason and ends the process, as NCCLCHECK /
 * CUDA_CHECK do there (communicator.h:40-67).  The one difference is the
 * tensor type: where the reference takes singa::Tensor, these methods take a
 * TensorRef - what the reference reads from a Tensor on this path:
 *     TensorRef{t.block()->mutable_data(), t.Size(), t.data_type() == kFloat16}
 * and the stream the caller's kernels run on (the reference's ctx->stream).
 * A maintainer's adapter inside libsinga is therefore three lines per method
 * (build the refs, call, done); singa_b200/adapter/communicator.cc is that
 * adapter, written on singa::Tensor and Device::Exec. */
#ifndef SGB_COMMUNICATOR_HPP_
#define SGB_COMMUNICATOR_HPP_

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "sgb.h"

namespace sgb {

struct TensorRef {
  void* data;      /* device pointer */
  size_t size;     /* elements */
  bool half;       /* fp16 data (synch / fusedSynch only) */
};

/* communicator.h:69-74.  The id is opaque bytes of sgb_comm_unique_id_bytes(). */
class NcclIdHolder {
 public:
  std::vector<unsigned char> id;
  NcclIdHolder() : id(sgb_comm_unique_id_bytes()) { check(sgb_comm_get_unique_id(id.data()), "ncclGetUniqueId"); }
  explicit NcclIdHolder(const std::vector<unsigned char>& bytes) : id(bytes) {}

  static void check(int status, const char* what) {
    if (status != SGB_OK) {
      std::fprintf(stderr, "Failed, %s: %s (cuda %d, nccl %d)\n", what, sgb_status_string(status),
                   sgb_last_cuda_error(), sgb_last_nccl_error());
      std::exit(EXIT_FAILURE);
    }
  }
};

class Communicator {
 public:
  int global_rank;
  int world_size;
  int local_rank;

  /* communicator.h:83: one process per GPU; `size` = elements of the staging buffers. */
  Communicator(int local_rank_, int world_size_, const NcclIdHolder& holder, size_t size)
      : global_rank(local_rank_), world_size(world_size_), local_rank(local_rank_) {
    NcclIdHolder::check(sgb_comm_create(&comm_, global_rank, world_size, holder.id.data(), size), "Communicator");
  }
  ~Communicator() { sgb_comm_destroy(comm_); }
  Communicator(const Communicator&) = delete;
  Communicator& operator=(const Communicator&) = delete;

  /* In-place all-reduce (sum) of one tensor. */
  void synch(TensorRef t, void* stream) {
    NcclIdHolder::check(sgb_comm_synch(comm_, t.data, t.size, t.half, stream), "synch");
  }
  /* send == false stages the tensors of a bucket; send == true reduces what was staged. */
  void fusedSynch(const std::vector<TensorRef>& t, void* stream, bool send = true) {
    table(t);
    NcclIdHolder::check(sgb_comm_fused_synch(comm_, ptrs_.data(), sizes_.data(), t.size(),
                                             !t.empty() && t[0].half, send, stream), "fusedSynch");
  }
  /* fp32 tensors carried as fp16 on the wire. */
  void synchHalf(TensorRef t, void* stream) {
    NcclIdHolder::check(sgb_comm_synch_half(comm_, static_cast<float*>(t.data), t.size, stream), "synchHalf");
  }
  void fusedSynchHalf(const std::vector<TensorRef>& t, void* stream, bool send = true) {
    table(t);
    NcclIdHolder::check(sgb_comm_fused_synch_half(comm_, ptrs_.data(), sizes_.data(), t.size(), send, stream),
                        "fusedSynchHalf");
  }
  /* Threshold (topK == false) or top-K sparsified exchange; `accumulation` is
   * the residual buffer of the same total size, or NULL for the overloads
   * without residual correction. */
  void fusedSparsification(const std::vector<TensorRef>& t, float* accumulation, float sparsThreshold, bool topK,
                           void* stream) {
    table(t);
    NcclIdHolder::check(sgb_comm_sparsification(comm_, ptrs_.data(), sizes_.data(), t.size(), accumulation,
                                                sparsThreshold, topK, stream), "fusedSparsification");
  }
  void sparsification(TensorRef t, float* accumulation, float sparsThreshold, bool topK, void* stream) {
    fusedSparsification(std::vector<TensorRef>{t}, accumulation, sparsThreshold, topK, stream);
  }
  /* The caller's stream waits for everything the communicator has in flight. */
  void wait(void* stream) { NcclIdHolder::check(sgb_comm_wait(comm_, stream), "wait"); }

  sgb_comm* handle() const { return comm_; }

 private:
  void table(const std::vector<TensorRef>& t) {
    ptrs_.resize(t.size());
    sizes_.resize(t.size());
    for (size_t i = 0; i < t.size(); ++i) {
      ptrs_[i] = t[i].data;
      sizes_[i] = t[i].size;
    }
  }
  sgb_comm* comm_ = nullptr;
  std::vector<void*> ptrs_;
  std::vector<size_t> sizes_;
};

}  // namespace sgb

#endif  /* SGB_COMMUNICATOR_HPP_ */
