// Replacement for apache/singa's include/singa/io/communicator.h: the same two
// classes with the same PUBLIC members (the SWIG interface
// src/api/dist_communicator.i:33-60 reads exactly these), implemented over the
// communicator of libsgb.so (include/sgb.h, sgb_comm_*) instead of the
// reference's src/io/communicator.cc.  Put this directory in front of the
// reference's include/ on the include path, compile
// singa_b200/adapter/communicator.cc instead of src/io/communicator.cc, and
// the rest of libsinga (and its Python layer) is unchanged.
//
// Differences a caller can observe: sizes are size_t internally (the
// reference multiplies element counts as int); the MPI-bootstrapped
// constructor Communicator(int) needs an MPI build and aborts here; the
// threshold sparsifier returns the count the reference intends (its literal
// code counts over unspecified memory).
#ifndef SINGA_IO_COMMUNICATOR_H_
#define SINGA_IO_COMMUNICATOR_H_
#include "singa/singa_config.h"
#ifdef USE_DIST
#include <nccl.h>

#include <memory>
#include <vector>

#include "sgb.h"
#include "singa/core/tensor.h"

namespace singa {
using std::vector;

class NcclIdHolder {
 public:
  ncclUniqueId id;
  NcclIdHolder();
  ~NcclIdHolder();
};

class Communicator {
 public:
  int global_rank;
  int world_size;
  int local_rank;

  Communicator(int limit);
  Communicator(int local_rank, int world_size, const NcclIdHolder &holder, int size);
  ~Communicator();
  void synch(Tensor &t);
  void fusedSynch(vector<Tensor> &t, bool send = true);
  void synchHalf(Tensor &t);
  void fusedSynchHalf(vector<Tensor> &t, bool send = true);
  void fusedSparsification(vector<Tensor> &t, Tensor &accumulation, float sparsThreshold, bool topK);
  void fusedSparsification(vector<Tensor> &t, float sparsThreshold, bool topK);
  void sparsification(Tensor &t, Tensor &accumulation, float sparsThreshold, bool topK);
  void sparsification(Tensor &t, float sparsThreshold, bool topK);
  void wait();

 private:
  // Collects the blocks of the tensors of one call and of the calls staged
  // before it: the read / write lists handed to Device::Exec, from which the
  // graph scheduler derives its dependencies.
  void track(const vector<Tensor> &t);
  void submit(const char *name, std::function<void(Context *)> &&fn);
  void sparse(vector<Tensor> &t, Tensor *accumulation, float spars, bool topK, const char *name);

  sgb_comm *comm_ = nullptr;
  bool streams_bound_ = false;
  std::shared_ptr<Device> device_;
  std::vector<Block *> blocks_;       // blocks touched since the last flush
};

}  // namespace singa
#endif  // USE_DIST
#endif  // SINGA_IO_COMMUNICATOR_H_
