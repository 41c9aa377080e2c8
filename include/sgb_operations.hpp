/* C++ host-side mirror of SINGA's operation handles and free functions on the
 * backward path (src/model/operation/batchnorm.{h,cc}, pooling.{h,cc},
 * convolution.cc:684-702) over the C ABI of sgb.h.  Header only; needs no
 * CUDA or cuDNN header.
 *
 * Same names and argument ORDER as the reference functions; where those take
 * and return singa::Tensor, these take device pointers (inputs first, then
 * the outputs the reference would allocate, then workspace and stream).  The
 * handle classes carry the fields the reference's handles carry and compute
 * them by the same rules.  A failed call prints the reason and aborts - the
 * reference's CHECK / LOG(FATAL) convention. */
#ifndef SGB_OPERATIONS_HPP_
#define SGB_OPERATIONS_HPP_

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "sgb.h"

namespace sgb {

inline void check_op(int status, const char* what) {
  if (status != SGB_OK) {
    std::fprintf(stderr, "%s failed: %s (cuda error %d)\n", what, sgb_status_string(status), sgb_last_cuda_error());
    std::abort();
  }
}

/* BatchNormHandle / CudnnBatchNormHandle (batchnorm.cc:27-41, 261-285):
 * 4-D input -> spatial statistics per channel; 2-D input -> one statistic
 * per feature (height = width = 1, is_2d). */
class CudnnBatchNormHandle {
 public:
  float factor;
  size_t batchsize, channels, height, width;
  bool is_2d;
  CudnnBatchNormHandle(float momentum, const std::vector<size_t>& input_shape) : factor(momentum) {
    if (input_shape.size() != 4u && input_shape.size() != 2u) {
      std::fprintf(stderr, "The dimension of input should either be 4D or 2D.\n");
      std::abort();
    }
    batchsize = input_shape[0];
    channels = input_shape[1];
    is_2d = input_shape.size() == 2u;
    height = is_2d ? 1 : input_shape[2];
    width = is_2d ? 1 : input_shape[3];
  }
  size_t workspace_bytes() const {
    return sgb_bn_backward_workspace_bytes(static_cast<int>(batchsize), static_cast<int>(channels),
                                           static_cast<int>(height * width));
  }
};

/* GpuBatchNormForwardTraining (batchnorm.cc:287-329): y, and the saved mean /
 * inverse standard deviation that the backward consumes; running statistics
 * are updated in place with the handle's factor.  eps is what the reference
 * passes (CUDNN_BN_MIN_EPSILON: 0 with cuDNN 8 and later). */
inline void GpuBatchNormForwardTraining(const CudnnBatchNormHandle& h, const float* x, const float* bnScale,
                                        const float* bnBias, float* running_mean, float* running_var, float* y,
                                        float* mean, float* var, void* ws, size_t ws_bytes, void* stream,
                                        double eps = 0.0) {
  check_op(sgb_bn_forward_training_f32(x, bnScale, bnBias, running_mean, running_var, h.factor, static_cast<float>(eps), y, mean, var,
                                       static_cast<int>(h.batchsize), static_cast<int>(h.channels),
                                       static_cast<int>(h.height * h.width), ws, ws_bytes, stream),
           "GpuBatchNormForwardTraining");
}

/* GpuBatchNormBackward (batchnorm.cc:368-404): {dx, dbnScale, dbnBias}. */
inline void GpuBatchNormBackward(const CudnnBatchNormHandle& h, const float* dy, const float* x, const float* bnScale,
                                 const float* mean, const float* var, float* dx, float* dbnScale, float* dbnBias,
                                 void* ws, size_t ws_bytes, void* stream) {
  check_op(sgb_bn_backward_f32(x, dy, bnScale, mean, var, dx, dbnScale, dbnBias, static_cast<int>(h.batchsize),
                               static_cast<int>(h.channels), static_cast<int>(h.height * h.width), ws, ws_bytes,
                               stream),
           "GpuBatchNormBackward");
}

/* PoolingHandle / CudnnPoolingHandle (pooling.cc:27-52, 150-178). */
class CudnnPoolingHandle {
 public:
  int kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w;
  int batchsize, channels, height, width, pooled_height, pooled_width;
  bool is_max_pooling;
  CudnnPoolingHandle(const std::vector<int>& input_shape, const std::vector<int>& kernel_size,
                     const std::vector<int>& stride, const std::vector<int>& padding, bool is_max = true)
      : kernel_h(kernel_size[0]), kernel_w(kernel_size[1]), pad_h(padding[0]), pad_w(padding[1]),
        stride_h(stride[0]), stride_w(stride[1]), batchsize(input_shape[0]), channels(input_shape[1]),
        height(input_shape[2]), width(input_shape[3]), pooled_height(1), is_max_pooling(is_max) {
    if (stride_h > 0) pooled_height = (height + 2 * pad_h - kernel_h) / stride_h + 1;
    pooled_width = (width + 2 * pad_w - kernel_w) / stride_w + 1;
  }
};

/* GpuPoolingForward (pooling.cc:180-205). */
inline void GpuPoolingForward(const CudnnPoolingHandle& h, const float* x, float* y, void* stream) {
  const int st = h.is_max_pooling
                     ? sgb_maxpool_forward_f32(x, y, h.batchsize, h.channels, h.height, h.width, h.kernel_h,
                                               h.kernel_w, h.pad_h, h.pad_w, h.stride_h, h.stride_w, stream)
                     : sgb_avgpool_forward_f32(x, y, h.batchsize, h.channels, h.height, h.width, h.kernel_h,
                                               h.kernel_w, h.pad_h, h.pad_w, h.stride_h, h.stride_w, stream);
  check_op(st, "GpuPoolingForward");
}

/* GpuPoolingBackward (pooling.cc:207-226): dx from (dy, x, y). */
inline void GpuPoolingBackward(const CudnnPoolingHandle& h, const float* dy, const float* x, const float* y,
                               float* dx, void* stream) {
  const int st = h.is_max_pooling
                     ? sgb_maxpool_backward_f32(x, y, dy, dx, h.batchsize, h.channels, h.height, h.width,
                                                h.kernel_h, h.kernel_w, h.pad_h, h.pad_w, h.stride_h, h.stride_w,
                                                stream)
                     : sgb_avgpool_backward_f32(dy, dx, h.batchsize, h.channels, h.height, h.width, h.kernel_h,
                                                h.kernel_w, h.pad_h, h.pad_w, h.stride_h, h.stride_w, stream);
  check_op(st, "GpuPoolingBackward");
}

/* Forward partner with an arg-max record (one byte per window) and the backward
 * that consumes only dy and that record; max pooling only.  No reference
 * counterpart: an optional pair for a _Pooling2d that keeps the record. */
inline void GpuPoolingForwardArgmax(const CudnnPoolingHandle& h, const float* x, float* y, unsigned char* argmax,
                                    void* stream) {
  check_op(sgb_maxpool_forward_argmax_f32(x, y, argmax, h.batchsize, h.channels, h.height, h.width, h.kernel_h,
                                          h.kernel_w, h.pad_h, h.pad_w, h.stride_h, h.stride_w, stream),
           "GpuPoolingForwardArgmax");
}
inline void GpuPoolingBackwardArgmax(const CudnnPoolingHandle& h, const float* dy, const unsigned char* argmax,
                                     float* dx, void* stream) {
  check_op(sgb_maxpool_backward_argmax_f32(dy, argmax, dx, h.batchsize, h.channels, h.height, h.width, h.kernel_h,
                                           h.kernel_w, h.pad_h, h.pad_w, h.stride_h, h.stride_w, stream),
           "GpuPoolingBackwardArgmax");
}

/* GpuConvBackwardb (convolution.cc:684-702): db[c] = sum over n, h, w of dy. */
inline void GpuConvBackwardb(const float* dy, float* db, int batchsize, int channels, int out_h, int out_w, void* ws,
                             size_t ws_bytes, void* stream) {
  check_op(sgb_conv_bias_backward_f32(dy, db, batchsize, channels, out_h * out_w, ws, ws_bytes, stream),
           "GpuConvBackwardb");
}

}  // namespace sgb

#endif  /* SGB_OPERATIONS_HPP_ */
