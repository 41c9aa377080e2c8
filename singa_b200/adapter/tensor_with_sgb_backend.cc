// Builds apache/singa's src/core/tensor/tensor.cc with this repository's CUDA
// back end in place of the reference's.  tensor.cc includes the back-end
// headers through relative paths ("./tensor_math_cuda.h"), which always
// resolve next to tensor.cc itself; including the replacement FIRST claims the
// shared include guard, so the reference's header contributes nothing when
// tensor.cc reaches it.  In an actual SINGA tree the replacement header simply
// takes the place of src/core/tensor/tensor_math_cuda.h and this file is not
// needed.  The include path must contain the reference's src/core/tensor.
#include "singa/core/tensor.h"
// tensor_math.h declares the generic templates the specialisations attach to
#include "tensor_math.h"
#include "tensor_math_cuda.h"  // this directory: singa_b200/adapter
#include "tensor.cc"           // the reference's src/core/tensor/tensor.cc
