// extern "C" doors into apache/singa's own core library compiled for its
// lang::Cpp (CPU) back end (oracle/ref_core_build.py).  TEST INFRASTRUCTURE
// ONLY: everything below runs on singa::Tensor objects through the reference's
// public C++ functions, in the order its Python autograd issues them, so the
// checker can (a) time the reference's CPU path on the MLP training step of
// benchmark configuration 1 and (b) pin the CPU restatement in oracle.c against
// the code it restates.
//
// Call sequences followed (apache/singa, python/singa):
//   Linear forward    autograd.py:603-610 (Mult) + :682-691 (AddRow)
//   ReLU              autograd.py:421-439 (ReLU / ReLUBackward)
//   loss head         autograd.py:1312-1322 (SoftMax, CrossEntropyFwd, SumAll, /N;
//                     SoftmaxCrossEntropyBwd, /N)
//   Linear backward   autograd.py:613-622 (two Mult on transposed views),
//                     :696-709 (Sum over axis 0)
//   SGD with momentum opt.py:269-310 (buf *= m; Axpy(1, g, buf); Axpy(-lr, buf, p))
#include <memory>
#include <vector>

#include "singa/core/device.h"
#include "singa/core/tensor.h"

using singa::Shape;
using singa::Tensor;

namespace {

struct Mlp {
  int batch = 0;
  std::vector<int> dims;
  std::vector<Tensor> W, b, mW, mb;
  float lr = 0.05f, momentum = 0.9f;
};

Tensor from_host(const float* src, const Shape& shape) {
  Tensor t(shape, singa::kFloat32);
  t.CopyDataFromHostPtr(src, t.Size());
  return t;
}

void sgd(Mlp* m, Tensor* param, Tensor grad, Tensor* buf) {
  if (m->momentum != 0.0f) {
    *buf *= m->momentum;
    singa::Axpy(1.0f, grad, buf);
    grad = *buf;
  }
  singa::Axpy(-m->lr, grad, param);
}

}  // namespace

extern "C" {

void* refcore_mlp_create(int batch, const int* dims, int ndims, float lr, float momentum) {
  Mlp* m = new Mlp();
  m->batch = batch;
  m->dims.assign(dims, dims + ndims);
  m->lr = lr;
  m->momentum = momentum;
  for (int i = 0; i + 1 < ndims; ++i) {
    m->W.emplace_back(Shape{static_cast<size_t>(dims[i]), static_cast<size_t>(dims[i + 1])});
    m->b.emplace_back(Shape{static_cast<size_t>(dims[i + 1])});
    m->mW.emplace_back(m->W.back().shape());
    m->mb.emplace_back(m->b.back().shape());
    m->W.back().SetValue(0.0f);
    m->b.back().SetValue(0.0f);
    m->mW.back().SetValue(0.0f);
    m->mb.back().SetValue(0.0f);
  }
  return m;
}

void refcore_mlp_destroy(void* h) { delete static_cast<Mlp*>(h); }

// which: 0 weight, 1 bias, 2 weight moment, 3 bias moment
static Tensor* pick(Mlp* m, int layer, int which) {
  std::vector<Tensor>* v = which == 0 ? &m->W : which == 1 ? &m->b : which == 2 ? &m->mW : &m->mb;
  return &(*v)[layer];
}

void refcore_mlp_set(void* h, int layer, int which, const float* src) {
  Tensor* t = pick(static_cast<Mlp*>(h), layer, which);
  t->CopyDataFromHostPtr(src, t->Size());
}

void refcore_mlp_get(void* h, int layer, int which, float* dst) {
  Tensor* t = pick(static_cast<Mlp*>(h), layer, which);
  t->GetValue(dst, t->Size());
}

// One forward + backward + SGD step; returns the mean loss.  When grads_out is
// not NULL it receives, layer by layer from the LAST layer to the first, the
// bias gradient followed by the weight gradient (the order they are produced).
float refcore_mlp_step(void* h, const float* x_host, const int* labels, float* grads_out) {
  Mlp* m = static_cast<Mlp*>(h);
  const size_t B = static_cast<size_t>(m->batch);
  const int L = static_cast<int>(m->W.size());
  Tensor x = from_host(x_host, Shape{B, static_cast<size_t>(m->dims[0])});
  Tensor t(Shape{B}, singa::kInt);
  t.CopyDataFromHostPtr(labels, B);
  // forward
  std::vector<Tensor> layer_in(L), relu_in(L);
  Tensor cur = x;
  for (int i = 0; i < L; ++i) {
    layer_in[i] = cur;
    Tensor y = singa::Mult(cur, m->W[i]);
    singa::AddRow(m->b[i], &y);
    if (i + 1 < L) {
      relu_in[i] = y;
      cur = singa::ReLU(y);
    } else {
      cur = y;
    }
  }
  Tensor p = singa::SoftMax(cur);
  Tensor per_sample = singa::CrossEntropyFwd(p, t);
  Tensor loss = singa::SumAll(per_sample);
  loss /= static_cast<float>(B);
  float loss_value = 0.0f;
  loss.GetValue(&loss_value, 1);
  // backward
  Tensor dy = singa::SoftmaxCrossEntropyBwd(p, t);
  dy /= static_cast<float>(B);
  float* out = grads_out;
  for (int i = L - 1; i >= 0; --i) {
    Tensor db = singa::Sum(dy, 0);
    Tensor dW = singa::Mult(singa::Transpose(layer_in[i]), dy);
    Tensor dx;
    if (i > 0) dx = singa::Mult(dy, singa::Transpose(m->W[i]));
    if (out) {
      db.GetValue(out, db.Size());
      out += db.Size();
      dW.GetValue(out, dW.Size());
      out += dW.Size();
    }
    sgd(m, &m->b[i], db, &m->mb[i]);
    sgd(m, &m->W[i], dW, &m->mW[i]);
    if (i > 0) dy = singa::ReLUBackward(dx, relu_in[i - 1]);
  }
  return loss_value;
}

// The same step restricted to the backward + update hot path: the contractions
// (the three Mult calls per layer) are left out and their outputs - the
// activation gradients dgrad[i] = dy W_i^T and the weight gradients wgrad[i] -
// are supplied by the caller as stand-ins, exactly as the GPU executor's plan
// for this configuration does.  relu_x[i] is the stored input of ReLU i.
// Arrays are indexed by layer; dgrad[0] is unused.  Returns the mean loss.
float refcore_mlp_hot_path_step(void* h, const float* logits, const int* labels, const float* const* relu_x,
                                const float* const* dgrad, const float* const* wgrad) {
  Mlp* m = static_cast<Mlp*>(h);
  const size_t B = static_cast<size_t>(m->batch);
  const int L = static_cast<int>(m->W.size());
  Tensor t(Shape{B}, singa::kInt);
  t.CopyDataFromHostPtr(labels, B);
  Tensor z = from_host(logits, Shape{B, static_cast<size_t>(m->dims[L])});
  Tensor p = singa::SoftMax(z);
  Tensor per_sample = singa::CrossEntropyFwd(p, t);
  Tensor loss = singa::SumAll(per_sample);
  loss /= static_cast<float>(B);
  float loss_value = 0.0f;
  loss.GetValue(&loss_value, 1);
  Tensor dy = singa::SoftmaxCrossEntropyBwd(p, t);
  dy /= static_cast<float>(B);
  for (int i = L - 1; i >= 0; --i) {
    Tensor db = singa::Sum(dy, 0);
    Tensor dW = from_host(wgrad[i], m->W[i].shape());
    sgd(m, &m->b[i], db, &m->mb[i]);
    sgd(m, &m->W[i], dW, &m->mW[i]);
    if (i > 0) {
      const Shape s{B, static_cast<size_t>(m->dims[i])};
      dy = singa::ReLUBackward(from_host(dgrad[i], s), from_host(relu_x[i - 1], s));
    }
  }
  return loss_value;
}

// ------------------------------------------------ single operations (cross-checks)
void refcore_relu_backward(const float* dy, const float* x, float* dx, size_t n) {
  Tensor a = from_host(dy, Shape{n}), b = from_host(x, Shape{n});
  Tensor r = singa::ReLUBackward(a, b);
  r.GetValue(dx, n);
}

void refcore_softmax(const float* x, float* y, size_t rows, size_t cols) {
  Tensor a = from_host(x, Shape{rows, cols});
  Tensor r = singa::SoftMax(a);
  r.GetValue(y, rows * cols);
}

void refcore_cross_entropy(const float* p, const int* t, float* loss, size_t rows, size_t cols) {
  Tensor a = from_host(p, Shape{rows, cols});
  Tensor lab(Shape{rows}, singa::kInt);
  lab.CopyDataFromHostPtr(t, rows);
  Tensor r = singa::CrossEntropyFwd(a, lab);
  r.GetValue(loss, rows);
}

void refcore_softmax_cross_entropy_bwd(const float* p, const int* t, float* grad, size_t rows, size_t cols) {
  Tensor a = from_host(p, Shape{rows, cols});
  Tensor lab(Shape{rows}, singa::kInt);
  lab.CopyDataFromHostPtr(t, rows);
  Tensor r = singa::SoftmaxCrossEntropyBwd(a, lab);
  r.GetValue(grad, rows * cols);
}

// Sum over axis 0 of a rows x cols matrix: the bias-gradient reduction.
void refcore_sum_axis0(const float* m, float* v, size_t rows, size_t cols) {
  Tensor a = from_host(m, Shape{rows, cols});
  Tensor r = singa::Sum(a, 0);
  r.GetValue(v, cols);
}

float refcore_sum_all(const float* x, size_t n) {
  Tensor a = from_host(x, Shape{n});
  Tensor r = singa::SumAll(a);
  float v = 0.0f;
  r.GetValue(&v, 1);
  return v;
}

// One SGD step with momentum and weight decay on flat arrays (opt.py:269-310).
void refcore_sgd(float* param, const float* grad, float* moment, size_t n, float lr, float momentum,
                 float weight_decay) {
  Tensor p = from_host(param, Shape{n}), g = from_host(grad, Shape{n}), b = from_host(moment, Shape{n});
  if (weight_decay != 0.0f) singa::Axpy(weight_decay, p, &g);
  if (momentum != 0.0f) {
    b *= momentum;
    singa::Axpy(1.0f, g, &b);
    g = b;
  }
  singa::Axpy(-lr, g, &p);
  p.GetValue(param, n);
  b.GetValue(moment, n);
}

}  // extern "C"
