/* The handful of CBLAS entry points apache/singa's lang::Cpp back end calls
 * (src/core/tensor/tensor_math_cpp.h: sgemm, sgemv, saxpy, sdot, sscal, snrm2,
 * sasum, isamax), declared here because no CBLAS is installed where the
 * comparator is built; ref_cblas.c implements them with plain OpenMP loops.
 * TEST INFRASTRUCTURE ONLY. */
#ifndef SGB_REF_CBLAS_H_
#define SGB_REF_CBLAS_H_
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
typedef CBLAS_ORDER CBLAS_LAYOUT;

void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, float alpha,
                 const float *A, int lda, const float *B, int ldb, float beta, float *C, int ldc);
void cblas_sgemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int M, int N, float alpha, const float *A, int lda,
                 const float *X, int incX, float beta, float *Y, int incY);
void cblas_saxpy(int n, float alpha, const float *X, int incX, float *Y, int incY);
float cblas_sdot(int n, const float *X, int incX, const float *Y, int incY);
void cblas_sscal(int n, float alpha, float *X, int incX);
float cblas_snrm2(int n, const float *X, int incX);
float cblas_sasum(int n, const float *X, int incX);
size_t cblas_isamax(int n, const float *X, int incX);
#ifdef __cplusplus
}
#endif
#endif
