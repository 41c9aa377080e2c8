// cusparseSaxpyi (y[xInd[i] - base] += alpha * xVal[i]) was removed from
// cuSPARSE in CUDA 12; apache/singa's communicator still calls it
// (src/io/communicator.cc:715, 753, 803).  This header, force-included when
// that file is compiled for the checker, declares a stand-in with the removed
// routine's signature; saxpyi_compat.cu implements it with one scatter-add
// kernel on the handle's stream.  TEST INFRASTRUCTURE ONLY.
#ifndef SGB_REF_SAXPYI_COMPAT_H_
#define SGB_REF_SAXPYI_COMPAT_H_
#include <cusparse.h>
cusparseStatus_t cusparseSaxpyi(cusparseHandle_t handle, int nnz, const float* alpha, const float* xVal,
                                const int* xInd, float* y, cusparseIndexBase_t idxBase);
#endif
