// Implementation of the cusparseSaxpyi stand-in declared in saxpyi_compat.h.
// Indices within one call are assumed distinct (they are in the caller: one
// rank's selected gradient positions), so a plain read-modify-write suffices.
#include "saxpyi_compat.h"

namespace {
__global__ void saxpyi_kernel(int nnz, float alpha, const float* __restrict__ val, const int* __restrict__ ind,
                              float* __restrict__ y, int base) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nnz; i += gridDim.x * blockDim.x) {
    const int j = ind[i] - base;
    if (j >= 0) y[j] += alpha * val[i];
  }
}
}  // namespace

cusparseStatus_t cusparseSaxpyi(cusparseHandle_t handle, int nnz, const float* alpha, const float* xVal,
                                const int* xInd, float* y, cusparseIndexBase_t idxBase) {
  if (nnz <= 0) return CUSPARSE_STATUS_SUCCESS;
  cudaStream_t s = nullptr;
  if (cusparseGetStream(handle, &s) != CUSPARSE_STATUS_SUCCESS) return CUSPARSE_STATUS_INTERNAL_ERROR;
  const int block = 256;
  int grid = (nnz + block - 1) / block;
  if (grid > 148 * 16) grid = 148 * 16;
  saxpyi_kernel<<<grid, block, 0, s>>>(nnz, *alpha, xVal, xInd, y, idxBase == CUSPARSE_INDEX_BASE_ONE ? 1 : 0);
  return cudaGetLastError() == cudaSuccess ? CUSPARSE_STATUS_SUCCESS : CUSPARSE_STATUS_EXECUTION_FAILED;
}
