// singa::Communicator / singa::NcclIdHolder (declared in
// singa_b200/adapter/singa/io/communicator.h with the reference's public
// interface) over the sgb_comm_* C ABI.  Replaces apache/singa's
// src/io/communicator.cc.  Every entry point keeps the reference's shape:
// it returns at once after submitting ONE operation to the tensors' device
// through Device::Exec, named like the reference's dominant operation of that
// call ("Dist_s_fusedSynch_allreduce", "Dist_c1_fusedSynch_filling", ... -
// src/io/communicator.cc:253, 271, 300, 326, 364-412, 439-466, 478-556), with
// the tensors captured by value, so that graph mode buffers and replays it and
// the device's time profiling picks the stream the name selects.  The work
// runs on the Context's own side streams (ctx->s, ctx->c1, ctx->c2), ordered
// after ctx->stream by the library.
#include "singa/io/communicator.h"

#ifdef USE_DIST
#include <cstring>
#include <functional>

namespace singa {
namespace {
void check(int status, const char *what) {
  if (status != SGB_OK)
    LOG(FATAL) << what << ": " << sgb_status_string(status) << " (status " << status << ", NCCL "
               << sgb_last_nccl_error() << ", CUDA " << sgb_last_cuda_error() << ")";
}

struct Table {
  std::vector<void *> ptrs;
  std::vector<size_t> sizes;
  explicit Table(const vector<Tensor> &t) {
    for (const Tensor &x : t) {
      ptrs.push_back(x.block()->mutable_data());
      sizes.push_back(x.Size());
    }
  }
};
}  // namespace

NcclIdHolder::NcclIdHolder() {
  static_assert(sizeof(ncclUniqueId) >= 1, "");
  CHECK_EQ(sgb_comm_unique_id_bytes(), static_cast<int>(sizeof(ncclUniqueId)));
  check(sgb_comm_get_unique_id(&id), "sgb_comm_get_unique_id");
}
NcclIdHolder::~NcclIdHolder() {}

Communicator::Communicator(int limit) {
  (void)limit;
  LOG(FATAL) << "Communicator(int): the MPI bootstrap needs an MPI build; create the communicator from an "
                "NcclIdHolder shared by the ranks instead";
}

Communicator::Communicator(int local_rank, int world_size, const NcclIdHolder &holder, int size) {
  this->local_rank = local_rank;
  this->global_rank = local_rank;
  this->world_size = world_size;
  CUDA_CHECK(cudaSetDevice(local_rank));
  check(sgb_comm_create(&comm_, local_rank, world_size, &holder.id, static_cast<size_t>(size)), "sgb_comm_create");
}

Communicator::~Communicator() {
  if (comm_) sgb_comm_destroy(comm_);
}

void Communicator::track(const vector<Tensor> &t) {
  CHECK_GT(t.size(), 0u);
  device_ = t[0].device();
  for (const Tensor &x : t) blocks_.push_back(x.block());
}

void Communicator::submit(const char *name, std::function<void(Context *)> &&fn) {
  sgb_comm *c = comm_;
  bool *bound = &streams_bound_;
  device_->Exec(
      [c, bound, fn](Context *ctx) mutable {
        if (!*bound) {   // first operation: adopt the device's side streams
          check(sgb_comm_use_streams(c, ctx->s, ctx->c1, ctx->c2), "sgb_comm_use_streams");
          *bound = true;
        }
        fn(ctx);
      },
      blocks_, blocks_, name);
}

void Communicator::wait() {
  if (!device_) return;          // nothing was ever submitted
  sgb_comm *c = comm_;
  device_->Exec([c](Context *ctx) mutable { check(sgb_comm_wait(c, ctx->stream), "sgb_comm_wait"); }, blocks_, blocks_,
                "Waiting");
  blocks_.clear();
}

void Communicator::synch(Tensor &t) {
  track({t});
  sgb_comm *c = comm_;
  Tensor held = t;
  submit("Dist_s_synch_allreduce", [c, held](Context *ctx) mutable {
    check(sgb_comm_synch(c, held.block()->mutable_data(), held.Size(), held.data_type() == kFloat16 ? 1 : 0,
                         ctx->stream),
          "sgb_comm_synch");
  });
}

void Communicator::fusedSynch(vector<Tensor> &t, bool send) {
  track(t);
  sgb_comm *c = comm_;
  vector<Tensor> held = t;
  const int is_half = t[0].data_type() == kFloat16 ? 1 : 0;
  submit(send ? "Dist_s_fusedSynch_allreduce" : "Dist_c1_fusedSynch_filling", [c, held, is_half, send](Context *ctx) mutable {
    Table tab(held);
    check(sgb_comm_fused_synch(c, tab.ptrs.data(), tab.sizes.data(), tab.ptrs.size(), is_half, send ? 1 : 0,
                               ctx->stream),
          "sgb_comm_fused_synch");
  });
}

void Communicator::synchHalf(Tensor &t) {
  CHECK_EQ(static_cast<int>(t.data_type()), static_cast<int>(kFloat32))
      << "only fp32 tensors are converted to 16 bits for the transfer";
  track({t});
  sgb_comm *c = comm_;
  Tensor held = t;
  submit("Dist_s_synchHalf_allreduce", [c, held](Context *ctx) mutable {
    check(sgb_comm_synch_half(c, static_cast<float *>(held.block()->mutable_data()), held.Size(), ctx->stream),
          "sgb_comm_synch_half");
  });
}

void Communicator::fusedSynchHalf(vector<Tensor> &t, bool send) {
  CHECK_EQ(static_cast<int>(t[0].data_type()), static_cast<int>(kFloat32))
      << "only fp32 tensors are converted to 16 bits for the transfer";
  track(t);
  sgb_comm *c = comm_;
  vector<Tensor> held = t;
  submit(send ? "Dist_s_fusedSynchHalf_allreduce" : "Dist_c1_fusedSynchHalf_filling", [c, held, send](Context *ctx) mutable {
    Table tab(held);
    check(sgb_comm_fused_synch_half(c, tab.ptrs.data(), tab.sizes.data(), tab.ptrs.size(), send ? 1 : 0, ctx->stream),
          "sgb_comm_fused_synch_half");
  });
}

void Communicator::sparse(vector<Tensor> &t, Tensor *accumulation, float spars, bool topK, const char *name) {
  CHECK_EQ(static_cast<int>(t[0].data_type()), static_cast<int>(kFloat32)) << "sparsification is fp32 only";
  track(t);
  if (accumulation) blocks_.push_back(accumulation->block());
  sgb_comm *c = comm_;
  vector<Tensor> held = t;
  Tensor acc = accumulation ? *accumulation : Tensor();
  const bool with_acc = accumulation != nullptr;
  submit(name, [c, held, acc, with_acc, spars, topK](Context *ctx) mutable {
    Table tab(held);
    float *a = with_acc ? static_cast<float *>(acc.block()->mutable_data()) : nullptr;
    check(sgb_comm_sparsification(c, tab.ptrs.data(), tab.sizes.data(), tab.ptrs.size(), a, spars, topK ? 1 : 0,
                                  ctx->stream),
          "sgb_comm_sparsification");
  });
}

void Communicator::sparsification(Tensor &t, Tensor &accumulation, float sparsThreshold, bool topK) {
  vector<Tensor> one{t};
  sparse(one, &accumulation, sparsThreshold, topK, "Dist_c1c2_sparsification");
}
void Communicator::sparsification(Tensor &t, float sparsThreshold, bool topK) {
  vector<Tensor> one{t};
  sparse(one, nullptr, sparsThreshold, topK, "Dist_c1c2_sparsification");
}
void Communicator::fusedSparsification(vector<Tensor> &t, Tensor &accumulation, float sparsThreshold, bool topK) {
  sparse(t, &accumulation, sparsThreshold, topK, "Dist_c1c2_fusedSparsification");
}
void Communicator::fusedSparsification(vector<Tensor> &t, float sparsThreshold, bool topK) {
  sparse(t, nullptr, sparsThreshold, topK, "Dist_c1c2_fusedSparsification");
}

}  // namespace singa
#endif  // USE_DIST
