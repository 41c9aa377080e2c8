/*
 * CPU oracle for the SINGA backward + gradient-update path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic
 * that apache/singa performs on the training backward path so that the CUDA
 * kernels of this repository can be checked against it.  Nothing on the
 * product path links, loads or calls it: only the test-suite, the smoke check
 * and the CPU leg of the benchmark do.
 *
 * Parity status: PINNED for the operations that the reference's own tests
 * hold golden vectors for (cross-entropy forward/backward, row softmax,
 * batch-norm statistics and backward, max/avg pooling forward/backward,
 * SGD/momentum/weight-decay, ReLU forward/backward, row/column sums) - see
 * tests/test_oracle_golden.py, which replays those vectors.  Pooling ties and
 * the top-K index set, which no reference test pins, are pinned instead
 * against the reference's own CUDA path run on a B200
 * (tests/test_vs_reference_cuda_gpu.py).  UNPINNED by the reference (it has no
 * test that could detect a difference) for: threshold compaction order,
 * residual accumulation over several steps and fp16 rounding; those follow
 * the reference source as cited below.
 *
 * Each function cites the reference file:line (paths inside apache/singa)
 * whose behaviour it follows.  Loops are OpenMP-parallel over independent
 * planes/rows so that the same code can serve as the timed CPU baseline.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------ */
/* Elementwise                                                         */
/* ------------------------------------------------------------------ */

/* ReLU forward, CUDA convention (x > 0 keeps x, everything else -> +0):
 * src/core/tensor/math_kernel.cu:235-241. */
void orc_relu_fwd_f32(size_t n, const float *x, float *y) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) y[i] = x[i] > 0.0f ? x[i] : 0.0f;
}

/* ReLU backward: dx = x > 0 ? dy : 0.
 * src/core/tensor/math_kernel.cu:253-259 (CUDA f32) and
 * src/core/tensor/tensor_math_cpp.h:446-451 (CPU) agree on this rule. */
void orc_relu_bwd_f32(size_t n, const float *dy, const float *x, float *dx) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) dx[i] = x[i] > 0.0f ? dy[i] : 0.0f;
}

/* Gradient join a += b (python/singa/autograd.py:204 ->
 * src/core/tensor/math_kernel.cu:111-117). */
void orc_add_inplace_f32(size_t n, float *a, const float *b) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) a[i] = a[i] + b[i];
}

/* x *= c (grad /= world is Div -> EltwiseMult(in, 1/x),
 * src/core/tensor/tensor_math.h:149-153). */
void orc_scale_inplace_f32(size_t n, float *a, float c) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) a[i] = a[i] * c;
}

/* ------------------------------------------------------------------ */
/* Softmax + cross entropy                                             */
/* ------------------------------------------------------------------ */

/* Row softmax, numerically "accurate" form exp(x - rowmax) / sum, which is
 * what both the cuDNN call (src/core/tensor/tensor_math_cuda.h:1274-1305) and
 * the native CPU code (src/core/tensor/tensor_math_cpp.h:360-380) compute.
 * The row maximum is seeded with the first element, as the CUDA RowMax does
 * (src/core/tensor/math_kernel.cu:488-499); the CPU RowMax seeds with 0 and
 * is wrong for all-negative rows, which is not reproduced. */
void orc_softmax_rows_f32(size_t nrow, size_t ncol, const float *x, float *y) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t r = 0; r < (ptrdiff_t)nrow; ++r) {
    const float *xr = x + (size_t)r * ncol;
    float *yr = y + (size_t)r * ncol;
    float m = xr[0];
    for (size_t c = 1; c < ncol; ++c) m = xr[c] > m ? xr[c] : m;
    double s = 0.0;
    for (size_t c = 0; c < ncol; ++c) s += exp((double)xr[c] - (double)m);
    for (size_t c = 0; c < ncol; ++c)
      yr[c] = (float)(exp((double)xr[c] - (double)m) / s);
  }
}

/* Per-sample cross entropy of probabilities p.
 * src/core/tensor/math_kernel.cu:539-562, tensor_math_cpp.h:1058-1088.
 * int_target: t holds one class index per sample; otherwise t is a
 * batch x dim integer weight array normalised by its row sum. */
void orc_ce_fwd_f32(int int_target, size_t batch, size_t dim, const float *p,
                    const int *t, float *loss) {
  for (size_t i = 0; i < batch; ++i) {
    if (int_target) {
      float pt = p[i * dim + (size_t)t[i]];
      loss[i] = -logf(pt > FLT_MIN ? pt : FLT_MIN);
    } else {
      float sum = 0.f;
      for (size_t j = 0; j < dim; ++j) sum += (float)t[i * dim + j];
      float l = 0.f;
      for (size_t j = 0; j < dim; ++j) {
        float pj = p[i * dim + j];
        l -= (float)t[i * dim + j] / sum * logf(pj > FLT_MIN ? pj : FLT_MIN);
      }
      loss[i] = l;
    }
  }
}

/* Softmax-cross-entropy backward: grad = p - target, computed out of place
 * (the reference clones p, src/core/tensor/tensor.cc:1717-1721, then edits
 * it in place, math_kernel.cu:564-586 / tensor_math_cpp.h:1090-1119). */
void orc_ce_bwd_f32(int int_target, size_t batch, size_t dim, const float *p,
                    const int *t, float *grad) {
  memcpy(grad, p, batch * dim * sizeof(float));
  for (size_t i = 0; i < batch; ++i) {
    if (int_target) {
      size_t pos = i * dim + (size_t)t[i];
      grad[pos] = p[pos] - 1.0f;
    } else {
      float sum = 0.f;
      for (size_t j = 0; j < dim; ++j) sum += (float)t[i * dim + j];
      for (size_t j = 0; j < dim; ++j)
        grad[i * dim + j] -= (float)t[i * dim + j] / sum;
    }
  }
}

/* ------------------------------------------------------------------ */
/* Reductions                                                          */
/* ------------------------------------------------------------------ */

/* SumRows: v[c] = sum over rows of M[r][c]  (bias gradient).
 * src/core/tensor/tensor.cc:1523-1538.  Double accumulation: the oracle is
 * the more exact side of a 1e-5 comparison. */
void orc_sum_rows_f32(size_t nrow, size_t ncol, const float *M, float *v) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t c = 0; c < (ptrdiff_t)ncol; ++c) {
    double s = 0.0;
    for (size_t r = 0; r < nrow; ++r) s += M[r * ncol + (size_t)c];
    v[c] = (float)s;
  }
}

/* SumColumns: v[r] = sum over columns of M[r][c].
 * src/core/tensor/tensor.cc:1508-1522. */
void orc_sum_columns_f32(size_t nrow, size_t ncol, const float *M, float *v) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t r = 0; r < (ptrdiff_t)nrow; ++r) {
    double s = 0.0;
    for (size_t c = 0; c < ncol; ++c) s += M[(size_t)r * ncol + c];
    v[r] = (float)s;
  }
}

/* SumAll (scalar loss): src/core/tensor/tensor.cc:1242-1254. */
float orc_sum_all_f32(size_t n, const float *x) {
  double s = 0.0;
  for (size_t i = 0; i < n; ++i) s += x[i];
  return (float)s;
}

/* Convolution bias gradient db[c] = sum over n,h,w of dy (NCHW).
 * src/model/operation/convolution.cc:684-702 (cudnnConvolutionBackwardBias). */
void orc_conv_bias_bwd_f32(size_t N, size_t C, size_t HW, const float *dy,
                           float *db) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t c = 0; c < (ptrdiff_t)C; ++c) {
    double s = 0.0;
    for (size_t n = 0; n < N; ++n) {
      const float *pl = dy + (n * C + (size_t)c) * HW;
      for (size_t i = 0; i < HW; ++i) s += pl[i];
    }
    db[c] = (float)s;
  }
}

/* ------------------------------------------------------------------ */
/* Batch normalisation                                                 */
/* ------------------------------------------------------------------ */

/* Forward-training statistics as the reference hands them to backward:
 * per-channel batch mean and the saved INVERSE standard deviation
 * 1/sqrt(biased_var + eps) (src/model/operation/batchnorm.cc:287-329; numpy
 * model in test/python/test_api.py:31-54).  eps is a parameter because the
 * reference passes CUDNN_BN_MIN_EPSILON, whose value depends on the cuDNN
 * version (1e-5 in cuDNN 7, 0 in cuDNN 9). */
void orc_bn_stats_spatial_f32(size_t N, size_t C, size_t HW, const float *x,
                              double eps, float *mean, float *invstd) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t c = 0; c < (ptrdiff_t)C; ++c) {
    double s = 0.0, ss = 0.0;
    const double M = (double)(N * HW);
    for (size_t n = 0; n < N; ++n) {
      const float *pl = x + (n * C + (size_t)c) * HW;
      for (size_t i = 0; i < HW; ++i) s += pl[i];
    }
    const double mu = s / M;
    for (size_t n = 0; n < N; ++n) {
      const float *pl = x + (n * C + (size_t)c) * HW;
      for (size_t i = 0; i < HW; ++i) {
        double d = pl[i] - mu;
        ss += d * d;
      }
    }
    mean[c] = (float)mu;
    invstd[c] = (float)(1.0 / sqrt(ss / M + eps));
  }
}

/* Spatial batch-norm backward with saved mean and saved inverse std
 * (src/model/operation/batchnorm.cc:368-404: cudnnBatchNormalizationBackward
 * with alpha=1, beta=0 for data and parameters):
 *   dbias[c]  = sum dy
 *   dscale[c] = sum dy * (x - mean) * r
 *   dx        = scale * r * (dy - dbias/M - (x - mean) * r * dscale / M)
 * with r = saved inverse std and M = N*H*W.  The per-activation mode is the
 * same formula with HW = 1 and C = the feature count. */
void orc_bn_bwd_spatial_f32(size_t N, size_t C, size_t HW, const float *x,
                            const float *dy, const float *scale,
                            const float *mean, const float *invstd, float *dx,
                            float *dscale, float *dbias) {
#pragma omp parallel for schedule(dynamic, 1)
  for (ptrdiff_t c = 0; c < (ptrdiff_t)C; ++c) {
    const double mu = mean[c], r = invstd[c], M = (double)(N * HW);
    double sdy = 0.0, sdyx = 0.0;
    for (size_t n = 0; n < N; ++n) {
      const size_t off = (n * C + (size_t)c) * HW;
      for (size_t i = 0; i < HW; ++i) {
        double g = dy[off + i];
        sdy += g;
        sdyx += g * ((double)x[off + i] - mu);
      }
    }
    const double ds = sdyx * r;
    dbias[c] = (float)sdy;
    dscale[c] = (float)ds;
    const double k = (double)scale[c] * r;
    const double a = sdy / M, b = ds * r / M;
    for (size_t n = 0; n < N; ++n) {
      const size_t off = (n * C + (size_t)c) * HW;
      for (size_t i = 0; i < HW; ++i)
        dx[off + i] =
            (float)(k * ((double)dy[off + i] - a - ((double)x[off + i] - mu) * b));
    }
  }
}

/* ------------------------------------------------------------------ */
/* Pooling (NCHW)                                                      */
/* ------------------------------------------------------------------ */

/* Output extent: src/model/operation/pooling.cc:46-51. */
int orc_pool_out(int in, int k, int pad, int stride) {
  return (in + 2 * pad - k) / stride + 1;
}

/* Max pooling forward; padding never wins (window clipped to the image),
 * the FIRST maximum in raster order is kept (strict '>'), as in
 * src/model/layer/pooling.cc:162-207.  argmax (may be NULL) receives the
 * flat h*W+w index inside the plane. */
void orc_maxpool_fwd_f32(int N, int C, int H, int W, int kh, int kw, int ph,
                         int pw, int sh, int sw, const float *x, float *y,
                         int *argmax) {
  const int OH = orc_pool_out(H, kh, ph, sh), OW = orc_pool_out(W, kw, pw, sw);
#pragma omp parallel for schedule(static)
  for (ptrdiff_t pl = 0; pl < (ptrdiff_t)N * C; ++pl) {
    const float *xp = x + (size_t)pl * H * W;
    float *yp = y + (size_t)pl * OH * OW;
    int *ap = argmax ? argmax + (size_t)pl * OH * OW : NULL;
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        int h0 = oh * sh - ph, w0 = ow * sw - pw;
        int h1 = h0 + kh < H ? h0 + kh : H, w1 = w0 + kw < W ? w0 + kw : W;
        if (h0 < 0) h0 = 0;
        if (w0 < 0) w0 = 0;
        float best = -FLT_MAX;
        int bi = -1;
        for (int h = h0; h < h1; ++h)
          for (int w = w0; w < w1; ++w)
            if (xp[h * W + w] > best) {
              best = xp[h * W + w];
              bi = h * W + w;
            }
        yp[oh * OW + ow] = best;
        if (ap) ap[oh * OW + ow] = bi;
      }
  }
}

/* Max pooling backward: every window adds its dy to the element that won it,
 * windows visited in raster order (src/model/layer/pooling.cc:209-233).  The
 * winner is recomputed from x with the first-maximum rule above; the CUDA
 * reference hands x, y and dy to cudnnPoolingBackward
 * (src/model/operation/pooling.cc:207-226), which also recomputes it. */
void orc_maxpool_bwd_f32(int N, int C, int H, int W, int kh, int kw, int ph,
                         int pw, int sh, int sw, const float *x,
                         const float *dy, float *dx) {
  const int OH = orc_pool_out(H, kh, ph, sh), OW = orc_pool_out(W, kw, pw, sw);
#pragma omp parallel for schedule(static)
  for (ptrdiff_t pl = 0; pl < (ptrdiff_t)N * C; ++pl) {
    const float *xp = x + (size_t)pl * H * W;
    const float *gp = dy + (size_t)pl * OH * OW;
    float *dp = dx + (size_t)pl * H * W;
    for (int i = 0; i < H * W; ++i) dp[i] = 0.f;
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        int h0 = oh * sh - ph, w0 = ow * sw - pw;
        int h1 = h0 + kh < H ? h0 + kh : H, w1 = w0 + kw < W ? w0 + kw : W;
        if (h0 < 0) h0 = 0;
        if (w0 < 0) w0 = 0;
        float best = -FLT_MAX;
        int bi = -1;
        for (int h = h0; h < h1; ++h)
          for (int w = w0; w < w1; ++w)
            if (xp[h * W + w] > best) {
              best = xp[h * W + w];
              bi = h * W + w;
            }
        if (bi >= 0) dp[bi] += gp[oh * OW + ow];
      }
  }
}

/* Average pooling, divisor = number of window cells inside the image
 * (CUDNN_POOLING_AVERAGE_COUNT_EXCLUDE_PADDING,
 * src/model/operation/pooling.cc:170-172). */
void orc_avgpool_fwd_f32(int N, int C, int H, int W, int kh, int kw, int ph,
                         int pw, int sh, int sw, const float *x, float *y) {
  const int OH = orc_pool_out(H, kh, ph, sh), OW = orc_pool_out(W, kw, pw, sw);
#pragma omp parallel for schedule(static)
  for (ptrdiff_t pl = 0; pl < (ptrdiff_t)N * C; ++pl) {
    const float *xp = x + (size_t)pl * H * W;
    float *yp = y + (size_t)pl * OH * OW;
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        int h0 = oh * sh - ph, w0 = ow * sw - pw;
        int h1 = h0 + kh < H ? h0 + kh : H, w1 = w0 + kw < W ? w0 + kw : W;
        if (h0 < 0) h0 = 0;
        if (w0 < 0) w0 = 0;
        double s = 0.0;
        for (int h = h0; h < h1; ++h)
          for (int w = w0; w < w1; ++w) s += xp[h * W + w];
        yp[oh * OW + ow] = (float)(s / (double)((h1 - h0) * (w1 - w0)));
      }
  }
}

void orc_avgpool_bwd_f32(int N, int C, int H, int W, int kh, int kw, int ph,
                         int pw, int sh, int sw, const float *dy, float *dx) {
  const int OH = orc_pool_out(H, kh, ph, sh), OW = orc_pool_out(W, kw, pw, sw);
#pragma omp parallel for schedule(static)
  for (ptrdiff_t pl = 0; pl < (ptrdiff_t)N * C; ++pl) {
    const float *gp = dy + (size_t)pl * OH * OW;
    float *dp = dx + (size_t)pl * H * W;
    for (int i = 0; i < H * W; ++i) dp[i] = 0.f;
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        int h0 = oh * sh - ph, w0 = ow * sw - pw;
        int h1 = h0 + kh < H ? h0 + kh : H, w1 = w0 + kw < W ? w0 + kw : W;
        if (h0 < 0) h0 = 0;
        if (w0 < 0) w0 = 0;
        const float share = gp[oh * OW + ow] / (float)((h1 - h0) * (w1 - w0));
        for (int h = h0; h < h1; ++h)
          for (int w = w0; w < w1; ++w) dp[h * W + w] += share;
      }
  }
}

/* ------------------------------------------------------------------ */
/* SGD with momentum, dampening, weight decay (python/singa/opt.py:269-310) */
/* ------------------------------------------------------------------ */

/* One SGD.apply on one parameter tensor, as the chain of fp32 BLAS-1 calls
 * the reference issues:
 *   g   += decay * p              (Axpy, if weight_decay != 0)
 *   buf  = buf * mom              (elementwise)
 *   buf += (1 - damp) * g         (Axpy)
 *   nesterov ? g += mom * buf : g = buf
 *   p   += (-lr) * g              (Axpy)
 * Each Axpy rounds once per element (fused multiply-add), as cuBLAS/CBLAS do.
 * With use_momentum == 0 the momentum lines are skipped. */
void orc_sgd_update_f32(size_t n, float *p, float *g, float *buf, float lr,
                        float mom, float damp, float decay, int use_momentum,
                        int nesterov) {
  const float alpha = 1.0f - damp;
  const float minus_lr = 0.0f - lr;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t i = 0; i < (ptrdiff_t)n; ++i) {
    float gi = g[i];
    if (decay != 0.0f) gi = fmaf(decay, p[i], gi);
    float step = gi;
    if (use_momentum) {
      float b = buf[i] * mom;
      b = fmaf(alpha, gi, b);
      buf[i] = b;
      step = nesterov ? fmaf(mom, b, gi) : b;
    }
    g[i] = gi;
    p[i] = fmaf(minus_lr, step, p[i]);
  }
}

/* ------------------------------------------------------------------ */
/* Sparsification arithmetic (src/io/communicator.cc:619-807)          */
/* ------------------------------------------------------------------ */

/* Threshold variant, intended semantics: with residual correction
 *   s = g + acc ; keep = |s| >= thr ; acc' = s - (keep ? s : 0)
 * payload = order-preserving list of (1-based index, value) of kept, non-zero
 * elements (communicator.cc:619-680; math_kernel.cu:628-642: an element whose
 * kept value is exactly 0 gets index 0 and is dropped by the compaction).
 * acc may be NULL (no correction).  Returns nnz. */
size_t orc_sparse_threshold_f32(size_t n, const float *g, float *acc, float thr,
                                int *idx_out, float *val_out) {
  size_t k = 0;
  for (size_t i = 0; i < n; ++i) {
    float s = acc ? g[i] + acc[i] : g[i];
    float kept = fabsf(s) >= thr ? s : 0.0f;
    if (acc) acc[i] = s - kept;
    if (kept != 0.0f) {
      idx_out[k] = (int)(i + 1);
      val_out[k] = kept;
      ++k;
    }
  }
  return k;
}

/* Dense reconstruction: dst[idx-1] += val for one rank's payload, ranks
 * applied in ascending order by the caller (communicator.cc:704-718). */
void orc_scatter_add_f32(size_t nnz, const int *idx, const float *val,
                         float *dst) {
  for (size_t j = 0; j < nnz; ++j)
    if (idx[j] > 0) dst[idx[j] - 1] += val[j];
}
