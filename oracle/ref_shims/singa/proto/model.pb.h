// Stand-in for the header protoc would generate from apache/singa's
// src/proto/model.proto, reduced to the one message the loss layer's interface
// names (include/singa/model/loss.h:34-42: `LossConf`, parsed from a string
// and handed to Setup, which the cross-entropy layer ignores) and the Phase
// flags its callers pass (model.proto:148-151).  TEST
// INFRASTRUCTURE ONLY: it lets the reference's own
// src/model/loss/softmax_cross_entropy.cc and test/singa/test_cross_entropy.cc
// compile unmodified into oracle/_ref/ (see oracle/ref_cuda_build.py).
#ifndef SINGA_PROTO_MODEL_PB_H_
#define SINGA_PROTO_MODEL_PB_H_
#include <string>

#include "singa/proto/core.pb.h"

namespace singa {

enum Phase { kTrain = 4, kEval = 8 };

class LossConf {
 public:
  bool ParseFromString(const std::string&) { return true; }
};

}  // namespace singa
#endif  // SINGA_PROTO_MODEL_PB_H_
