/* Plain OpenMP implementations of the CBLAS subset declared in cblas.h (row-
 * and column-major sgemm / sgemv, level-1 routines with unit or general
 * strides).  They stand in for the CBLAS library apache/singa links against
 * (OpenBLAS in its builds; not installed here), so that its lang::Cpp back end
 * can be compiled and timed on the host cores.  TEST INFRASTRUCTURE ONLY. */
#include "cblas.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* C = alpha * op(A) * op(B) + beta * C in row-major storage. */
static void sgemm_rowmajor(int ta, int tb, int M, int N, int K, float alpha, const float *A, int lda,
                           const float *B, int ldb, float beta, float *C, int ldc) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i) {
    float *c = C + (size_t)i * ldc;
    if (beta == 0.0f) {
      memset(c, 0, sizeof(float) * (size_t)N);
    } else if (beta != 1.0f) {
      for (int j = 0; j < N; ++j) c[j] *= beta;
    }
    if (!tb) {
      /* rank-1 updates over k: contiguous rows of B, vectorisable */
      for (int k = 0; k < K; ++k) {
        const float a = alpha * (ta ? A[(size_t)k * lda + i] : A[(size_t)i * lda + k]);
        const float *b = B + (size_t)k * ldb;
        for (int j = 0; j < N; ++j) c[j] += a * b[j];
      }
    } else {
      for (int j = 0; j < N; ++j) {
        const float *b = B + (size_t)j * ldb;
        float acc = 0.0f;
        if (!ta) {
          const float *a = A + (size_t)i * lda;
          for (int k = 0; k < K; ++k) acc += a[k] * b[k];
        } else {
          for (int k = 0; k < K; ++k) acc += A[(size_t)k * lda + i] * b[k];
        }
        c[j] += alpha * acc;
      }
    }
  }
}

void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, float alpha,
                 const float *A, int lda, const float *B, int ldb, float beta, float *C, int ldc) {
  const int a_t = ta != CblasNoTrans, b_t = tb != CblasNoTrans;
  if (order == CblasRowMajor) {
    sgemm_rowmajor(a_t, b_t, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  } else {
    /* column-major C (M x N) is row-major C^T (N x M) = op(B)^T op(A)^T */
    sgemm_rowmajor(b_t, a_t, N, M, K, alpha, B, ldb, A, lda, beta, C, ldc);
  }
}

void cblas_sgemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int M, int N, float alpha, const float *A, int lda,
                 const float *X, int incX, float beta, float *Y, int incY) {
  /* A is M x N in the given order; y = alpha * op(A) x + beta * y */
  int trans = ta != CblasNoTrans;
  int rows = M, cols = N;
  if (order == CblasColMajor) { /* a column-major M x N matrix is a row-major N x M one, transposed */
    trans = !trans;
    rows = N;
    cols = M;
  }
  if (!trans) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < rows; ++i) {
      const float *a = A + (size_t)i * lda;
      float acc = 0.0f;
      for (int j = 0; j < cols; ++j) acc += a[j] * X[(size_t)j * incX];
      float *y = Y + (size_t)i * incY;
      *y = alpha * acc + (beta == 0.0f ? 0.0f : beta * *y);
    }
  } else {
#pragma omp parallel for schedule(static)
    for (int j = 0; j < cols; ++j) {
      float acc = 0.0f;
      for (int i = 0; i < rows; ++i) acc += A[(size_t)i * lda + j] * X[(size_t)i * incX];
      float *y = Y + (size_t)j * incY;
      *y = alpha * acc + (beta == 0.0f ? 0.0f : beta * *y);
    }
  }
}

void cblas_saxpy(int n, float alpha, const float *X, int incX, float *Y, int incY) {
#pragma omp parallel for schedule(static) if (n > 65536)
  for (int i = 0; i < n; ++i) Y[(size_t)i * incY] += alpha * X[(size_t)i * incX];
}

float cblas_sdot(int n, const float *X, int incX, const float *Y, int incY) {
  float acc = 0.0f;
#pragma omp parallel for schedule(static) reduction(+ : acc) if (n > 65536)
  for (int i = 0; i < n; ++i) acc += X[(size_t)i * incX] * Y[(size_t)i * incY];
  return acc;
}

void cblas_sscal(int n, float alpha, float *X, int incX) {
#pragma omp parallel for schedule(static) if (n > 65536)
  for (int i = 0; i < n; ++i) X[(size_t)i * incX] *= alpha;
}

float cblas_snrm2(int n, const float *X, int incX) {
  double acc = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : acc) if (n > 65536)
  for (int i = 0; i < n; ++i) acc += (double)X[(size_t)i * incX] * X[(size_t)i * incX];
  return (float)sqrt(acc);
}

float cblas_sasum(int n, const float *X, int incX) {
  float acc = 0.0f;
#pragma omp parallel for schedule(static) reduction(+ : acc) if (n > 65536)
  for (int i = 0; i < n; ++i) acc += fabsf(X[(size_t)i * incX]);
  return acc;
}

size_t cblas_isamax(int n, const float *X, int incX) {
  size_t best = 0;
  float v = -1.0f;
  for (int i = 0; i < n; ++i) {
    const float a = fabsf(X[(size_t)i * incX]);
    if (a > v) {
      v = a;
      best = (size_t)i;
    }
  }
  return best;
}
