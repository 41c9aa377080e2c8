// Streaming batch-norm backward: host-side interface of bn_stream.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace sgb {

// How a (N, C, HW) problem is cut for the streaming kernel.  A channel's data
// is N runs of HW floats; a run is cut into P pieces of Lp floats, and S
// consecutive pieces (in (n, piece) order) form one work item.
struct BnStreamPlan {
  int P;        // pieces per plane; P * Lp == HW
  int Lp;       // floats per piece, a multiple of 4
  int S;        // pieces per item
  int parts;    // items per channel = ceil(N * P / S)
  int depth;    // CTAs resident per SM (one staging slot each)
  int arrays;   // tensors staged per item (x, dy [, ReLU input])
};

// True when the streaming kernel can take the problem (plane a multiple of 4
// floats, a piece fits a slot, C within the exchange table); fills `plan`.
// mask: 0 none, 1 ReLU input as floats, 2 ReLU bit record.
bool bn_stream_plan(int N, int C, int HW, int mask, BnStreamPlan* plan);

// Bytes of workspace the streaming kernel needs for its per-item partial sums.
size_t bn_stream_workspace_bytes(int N, int C, int HW);

// Launches the kernel.  All pointers 16-byte aligned; `relu` is the ReLU input
// (mask 1) or the bit record (mask 2), unused for mask 0; `partial` holds
// bn_stream_workspace_bytes.
int bn_stream_backward(int mask, const float* x, const float* dy, const void* relu, const float* scale,
                       const float* mean, const float* invstd, float* dx, float* dscale, float* dbias,
                       int N, int C, int HW, const BnStreamPlan& plan, void* partial, cudaStream_t s);

// Sticky fault word of the streaming kernel on the current device (0 = none):
// bit 0 a bounded wait ran out, bit 1 the exchange block was in use by
// another launch.  Synchronises the device.
int bn_stream_faults(unsigned* flags);

}  // namespace sgb
