// The cuDNN calls that the reference issues for batch-norm and pooling
// backward (apache/singa src/model/operation/batchnorm.cc:368-404 and
// pooling.cc:150-226), issued here from a small harness with the same
// descriptors, modes and alpha/beta so that the new kernels can be compared
// with what the reference's CUDA path computes on the same device buffers.
// TEST INFRASTRUCTURE ONLY (oracle/_ref/libref_cudnn.so, built by
// oracle/ref_build.py).  Every function returns the cudnnStatus_t (0 = ok).
#include <cudnn.h>

namespace {
cudnnHandle_t handle() {
  static cudnnHandle_t h = nullptr;
  if (!h) cudnnCreate(&h);
  return h;
}
}  // namespace

#define CK(call)                          \
  do {                                    \
    cudnnStatus_t s__ = (call);           \
    if (s__ != CUDNN_STATUS_SUCCESS) return static_cast<int>(s__); \
  } while (0)

extern "C" {

int refcudnn_version() { return static_cast<int>(cudnnGetVersion()); }

// spatial (4-D) or per-activation (hw == 1 with is_2d) batch-norm:
// forward-training produces saved mean / saved inverse std, backward consumes them.
int refcudnn_bn_forward_training(int is_2d, int N, int C, int H, int W, double eps, const float* x,
                                 const float* scale, const float* bias, float* y,
                                 float* running_mean, float* running_var, double factor,
                                 float* save_mean, float* save_invstd, void* stream) {
  cudnnSetStream(handle(), static_cast<cudaStream_t>(stream));
  cudnnTensorDescriptor_t sd, pd;
  CK(cudnnCreateTensorDescriptor(&sd));
  CK(cudnnCreateTensorDescriptor(&pd));
  CK(cudnnSetTensor4dDescriptor(sd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  CK(cudnnSetTensor4dDescriptor(pd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, 1, C, is_2d ? 1 : 1, is_2d ? 1 : 1));
  const float alpha = 1.0f, beta = 0.0f;
  const cudnnBatchNormMode_t mode = is_2d ? CUDNN_BATCHNORM_PER_ACTIVATION : CUDNN_BATCHNORM_SPATIAL;
  CK(cudnnBatchNormalizationForwardTraining(handle(), mode, &alpha, &beta, sd, x, sd, y, pd, scale, bias,
                                            factor, running_mean, running_var, eps, save_mean,
                                            save_invstd));
  cudnnDestroyTensorDescriptor(sd);
  cudnnDestroyTensorDescriptor(pd);
  return 0;
}

int refcudnn_bn_backward(int is_2d, int N, int C, int H, int W, double eps, const float* x,
                         const float* dy, const float* scale, const float* save_mean,
                         const float* save_invstd, float* dx, float* dscale, float* dbias,
                         void* stream) {
  cudnnSetStream(handle(), static_cast<cudaStream_t>(stream));
  cudnnTensorDescriptor_t sd, pd;
  CK(cudnnCreateTensorDescriptor(&sd));
  CK(cudnnCreateTensorDescriptor(&pd));
  CK(cudnnSetTensor4dDescriptor(sd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  CK(cudnnSetTensor4dDescriptor(pd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, 1, C, 1, 1));
  const float alpha = 1.0f, beta = 0.0f;
  const cudnnBatchNormMode_t mode = is_2d ? CUDNN_BATCHNORM_PER_ACTIVATION : CUDNN_BATCHNORM_SPATIAL;
  CK(cudnnBatchNormalizationBackward(handle(), mode, &alpha, &beta, &alpha, &beta, sd, x, sd, dy, sd, dx,
                                     pd, scale, dscale, dbias, eps, save_mean, save_invstd));
  cudnnDestroyTensorDescriptor(sd);
  cudnnDestroyTensorDescriptor(pd);
  return 0;
}

double refcudnn_bn_min_epsilon() { return CUDNN_BN_MIN_EPSILON; }

int refcudnn_pooling(int backward, int is_max, int N, int C, int H, int W, int OH, int OW, int kh,
                     int kw, int ph, int pw, int sh, int sw, const float* x, float* y,
                     const float* dy, float* dx, void* stream) {
  cudnnSetStream(handle(), static_cast<cudaStream_t>(stream));
  cudnnTensorDescriptor_t xd, yd;
  cudnnPoolingDescriptor_t pd;
  CK(cudnnCreateTensorDescriptor(&xd));
  CK(cudnnCreateTensorDescriptor(&yd));
  CK(cudnnCreatePoolingDescriptor(&pd));
  CK(cudnnSetTensor4dDescriptor(xd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  CK(cudnnSetTensor4dDescriptor(yd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, OH, OW));
  CK(cudnnSetPooling2dDescriptor(pd, is_max ? CUDNN_POOLING_MAX : CUDNN_POOLING_AVERAGE_COUNT_EXCLUDE_PADDING,
                                 CUDNN_PROPAGATE_NAN, kh, kw, ph, pw, sh, sw));
  const float alpha = 1.0f, beta = 0.0f;
  if (!backward) {
    CK(cudnnPoolingForward(handle(), pd, &alpha, xd, x, &beta, yd, y));
  } else {
    CK(cudnnPoolingBackward(handle(), pd, &alpha, yd, y, yd, dy, xd, x, &beta, xd, dx));
  }
  cudnnDestroyPoolingDescriptor(pd);
  cudnnDestroyTensorDescriptor(xd);
  cudnnDestroyTensorDescriptor(yd);
  return 0;
}

// The bias gradient of a convolution as the reference computes it
// (apache/singa src/model/operation/convolution.cc:684-702):
// cudnnConvolutionBackwardBias on the NCHW output gradient with a 1 x C x 1 x 1
// bias descriptor, alpha = 1, beta = 0.
int refcudnn_conv_bias_backward(int N, int C, int H, int W, const float* dy, float* db, void* stream) {
  cudnnSetStream(handle(), static_cast<cudaStream_t>(stream));
  cudnnTensorDescriptor_t yd, bd;
  CK(cudnnCreateTensorDescriptor(&yd));
  CK(cudnnCreateTensorDescriptor(&bd));
  CK(cudnnSetTensor4dDescriptor(yd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  CK(cudnnSetTensor4dDescriptor(bd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, 1, C, 1, 1));
  const float alpha = 1.0f, beta = 0.0f;
  CK(cudnnConvolutionBackwardBias(handle(), &alpha, yd, dy, &beta, bd, db));
  cudnnDestroyTensorDescriptor(yd);
  cudnnDestroyTensorDescriptor(bd);
  return 0;
}
}
