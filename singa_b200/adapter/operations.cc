// Replacement bodies for three functions of apache/singa's operation layer,
// with the reference's signatures on singa::Tensor and its handle classes, so
// that its Python autograd (through SWIG, src/api/model_operation.i:37-230)
// runs on them unchanged:
//
//   GpuBatchNormBackward   src/model/operation/batchnorm.cc:368-404
//                          (cudnnBatchNormalizationBackward)
//   GpuPoolingBackward     src/model/operation/pooling.cc:207-226
//                          (cudnnPoolingBackward)
//   GpuConvBackwardb       src/model/operation/convolution.cc:684-702
//                          (cudnnConvolutionBackwardBias)
//
// Each keeps the reference's contract: the results are NEW tensors laid out
// like the corresponding inputs (ResetLike), the work is submitted through
// Device::Exec with the same read / write block lists and operation name (the
// graph scheduler derives its dependencies and its profiling streams from
// them), the tensors are captured by value so their blocks outlive a buffered
// operation, and everything runs on ctx->stream.  The handle classes and the
// forward functions are the reference's own.  In an actual SINGA tree these
// bodies replace the three functions in place.
#include <vector>

#include "model/operation/batchnorm.h"
#include "model/operation/convolution.h"
#include "model/operation/pooling.h"
#include "sgb.h"
#include "singa/core/tensor.h"

#ifdef USE_CUDNN
namespace singa {
namespace {

void check(int status, const char* what) {
  if (status != SGB_OK) LOG(FATAL) << what << ": " << sgb_status_string(status) << " (status " << status << ")";
}

// Device scratch from the tensor's memory pool (the C ABI allocates nothing).
Tensor workspace(const Tensor& like, size_t bytes) {
  return Tensor(Shape{bytes / sizeof(float) + 64}, like.device(), kFloat32);
}

}  // namespace

/// {dx, dscale, dbias} of a training-mode batch normalisation from the saved
/// mean and saved inverse standard deviation (what the forward-training
/// function returns as "mean" and "var").
const std::vector<Tensor> GpuBatchNormBackward(const CudnnBatchNormHandle& cbnh, const Tensor& dy, const Tensor& x,
                                               const Tensor& bnScale, const Tensor& mean, const Tensor& var) {
  CHECK_EQ(dy.device()->lang(), kCuda);
  CHECK_EQ(x.device()->lang(), kCuda);
  CHECK_EQ(bnScale.device()->lang(), kCuda);
  CHECK_EQ(mean.device()->lang(), kCuda);
  CHECK_EQ(var.device()->lang(), kCuda);
  CHECK_EQ(static_cast<int>(x.data_type()), static_cast<int>(kFloat32)) << "batch-norm backward is fp32";

  Tensor dx, dscale, dbias;
  dx.ResetLike(dy);
  dscale.ResetLike(bnScale);
  dbias.ResetLike(bnScale);

  const int N = static_cast<int>(cbnh.batchsize), C = static_cast<int>(cbnh.channels);
  const int HW = static_cast<int>(cbnh.height * cbnh.width);
  const size_t ws_bytes = sgb_bn_backward_workspace_bytes(N, C, HW);
  Tensor ws = workspace(dy, ws_bytes);

  dx.device()->Exec(
      [=](Context* ctx) mutable {
        (void)cudaGetLastError();   // drop an error parked by an earlier unchecked call
        check(sgb_bn_backward_f32(static_cast<const float*>(x.block()->data()),
                                  static_cast<const float*>(dy.block()->data()),
                                  static_cast<const float*>(bnScale.block()->data()),
                                  static_cast<const float*>(mean.block()->data()),
                                  static_cast<const float*>(var.block()->data()),
                                  static_cast<float*>(dx.block()->mutable_data()),
                                  static_cast<float*>(dscale.block()->mutable_data()),
                                  static_cast<float*>(dbias.block()->mutable_data()), N, C, HW,
                                  ws.block()->mutable_data(), ws.Size() * sizeof(float), ctx->stream),
              "sgb_bn_backward_f32");
      },
      {x.block(), dy.block(), bnScale.block(), mean.block(), var.block()},
      {dx.block(), dscale.block(), dbias.block()}, "GpuBatchNormBackward");

  if (cbnh.is_2d) dx.Reshape(Shape{dx.shape().at(0), dx.shape().at(1)});
  return {dx, dscale, dbias};
}

/// dx of max pooling (the gradient goes to the first maximum of each window in
/// raster order) or of average pooling that excludes the padding.
Tensor GpuPoolingBackward(const CudnnPoolingHandle& cph, const Tensor& dy, const Tensor& x, const Tensor& y) {
  CHECK_EQ(dy.device()->lang(), kCuda);
  CHECK_EQ(dy.nDim(), 4u);
  CHECK_EQ(static_cast<int>(x.data_type()), static_cast<int>(kFloat32)) << "pooling backward is fp32";

  Tensor dx;
  dx.ResetLike(x);

  const bool is_max = cph.is_max_pooling;
  const int N = cph.batchsize, C = cph.channels, H = cph.height, W = cph.width;
  const int kh = cph.kernel_h, kw = cph.kernel_w, ph = cph.pad_h, pw = cph.pad_w, sh = cph.stride_h,
            sw = cph.stride_w;

  dx.device()->Exec(
      [=](Context* ctx) mutable {
        const float* g = static_cast<const float*>(dy.block()->data());
        float* out = static_cast<float*>(dx.block()->mutable_data());
        (void)cudaGetLastError();   // drop an error parked by an earlier unchecked call
        if (is_max)
          check(sgb_maxpool_backward_f32(static_cast<const float*>(x.block()->data()),
                                         static_cast<const float*>(y.block()->data()), g, out, N, C, H, W, kh, kw,
                                         ph, pw, sh, sw, ctx->stream),
                "sgb_maxpool_backward_f32");
        else
          check(sgb_avgpool_backward_f32(g, out, N, C, H, W, kh, kw, ph, pw, sh, sw, ctx->stream),
                "sgb_avgpool_backward_f32");
      },
      {dy.block(), y.block(), x.block()}, {dx.block()}, "GpuPoolingBackward");
  return dx;
}

/// db[c] = sum of dy over the batch and the spatial positions.  `b` only lends
/// its layout; the handle is not consulted (the shapes come from dy).
Tensor GpuConvBackwardb(const Tensor& dy, const Tensor& b, const CudnnConvHandle& cch) {
  (void)cch;
  CHECK_EQ(dy.device()->lang(), kCuda);
  CHECK_GE(dy.nDim(), 2u);

  Tensor db;
  db.ResetLike(b);

  const int N = static_cast<int>(dy.shape(0)), C = static_cast<int>(dy.shape(1));
  const int HW = static_cast<int>(dy.Size() / (dy.shape(0) * dy.shape(1)));
  const size_t ws_bytes = sgb_conv_bias_backward_workspace_bytes(N, C, HW);
  Tensor ws = workspace(dy, ws_bytes);

  dy.device()->Exec(
      [=](Context* ctx) mutable {
        (void)cudaGetLastError();
        check(sgb_conv_bias_backward_f32(static_cast<const float*>(dy.block()->data()),
                                         static_cast<float*>(db.block()->mutable_data()), N, C, HW,
                                         ws.block()->mutable_data(), ws.Size() * sizeof(float), ctx->stream),
              "sgb_conv_bias_backward_f32");
      },
      {dy.block()}, {db.block()}, "cudnnConvolutionBackwardBias");
  return db;
}

}  // namespace singa
#endif  // USE_CUDNN
