// singa_wrap (pybind11): the free functions on singa::Tensor that the SWIG
// interface exposes (src/api/core_tensor.i:180-391), under the same names.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <pybind11/stl_bind.h>

#include <vector>

#include "singa/core/tensor.h"

namespace py = pybind11;
using singa::Tensor;

PYBIND11_MAKE_OPAQUE(std::vector<singa::Tensor>);

namespace {
using Unary = Tensor (*)(const Tensor&);
using Pair = Tensor (*)(const Tensor&, const Tensor&);
using PairOut = void (*)(const Tensor&, const Tensor&, Tensor*);
using RowCol = void (*)(const Tensor&, Tensor*);
}  // namespace

void bind_math(py::module_& m) {
  m.def("CopyDataToFrom", &singa::CopyDataToFrom, py::arg("dst"), py::arg("src"), py::arg("num"),
        py::arg("src_offset") = 0, py::arg("dst_offset") = 0);
  m.def("RepeatDataToFrom", &singa::RepeatDataToFrom);
  m.def("Reshape", [](const Tensor& t, const std::vector<size_t>& s) { return singa::Reshape(t, s); });
  m.def("Contiguous", &singa::Contiguous);
  m.def("Transpose", [](const Tensor& t, const std::vector<size_t>& axes) { return singa::Transpose(t, axes); });
  m.def("DefaultTranspose", [](const Tensor& t) { return singa::Transpose(t); });

#define SGB_BIND_UNARY(Name) m.def(#Name, static_cast<Unary>(&singa::Name))
  SGB_BIND_UNARY(Abs);
  SGB_BIND_UNARY(Ceil);
  SGB_BIND_UNARY(Floor);
  SGB_BIND_UNARY(Round);
  SGB_BIND_UNARY(RoundE);
  SGB_BIND_UNARY(Exp);
  SGB_BIND_UNARY(Erf);
  SGB_BIND_UNARY(Log);
  SGB_BIND_UNARY(ReLU);
  SGB_BIND_UNARY(Sigmoid);
  SGB_BIND_UNARY(Sign);
  SGB_BIND_UNARY(Sqrt);
  SGB_BIND_UNARY(Square);
  SGB_BIND_UNARY(Cos);
  SGB_BIND_UNARY(Cosh);
  SGB_BIND_UNARY(Acos);
  SGB_BIND_UNARY(Acosh);
  SGB_BIND_UNARY(Sin);
  SGB_BIND_UNARY(Sinh);
  SGB_BIND_UNARY(Asin);
  SGB_BIND_UNARY(Asinh);
  SGB_BIND_UNARY(Tan);
  SGB_BIND_UNARY(Tanh);
  SGB_BIND_UNARY(Atan);
  SGB_BIND_UNARY(Atanh);
#undef SGB_BIND_UNARY

  m.def("ReLUBackward", static_cast<Pair>(&singa::ReLUBackward));
  m.def("Sum", [](const Tensor& t, int axis) { return singa::Sum(t, axis); });
  m.def("SumAsFloat", [](const Tensor& t) { return singa::Sum<float>(t); });
  m.def("SumAll", &singa::SumAll);
  m.def("Average", &singa::Average);
  m.def("SoftMax", [](const Tensor& t) { return singa::SoftMax(t); });
  m.def("SoftMax", [](const Tensor& t, int axis) { return singa::SoftMax(t, axis); });
  m.def("SoftMax", [](const Tensor& t, Tensor* out) { singa::SoftMax(t, out); });
  m.def("SoftMax", [](const Tensor& t, Tensor* out, int axis) { singa::SoftMax(t, out, axis); });
  m.def("SoftMaxBackward", &singa::SoftMaxBackward);

  m.def("Pow", [](const Tensor& b, const Tensor& e) { return singa::Pow(b, e); });
  m.def("PowWithRet", [](const Tensor& b, const Tensor& e, Tensor* out) { singa::Pow(b, e, out); });
  m.def("PowFloat", [](const Tensor& t, float x) { return singa::Pow(t, x); });
  m.def("PowFloatWithRet", [](const Tensor& t, float x, Tensor* out) { singa::Pow(t, x, out); });

  // comparisons: tensor with tensor, tensor with float
  m.def("__lt__", [](const Tensor& a, const Tensor& b) { return a < b; });
  m.def("__le__", [](const Tensor& a, const Tensor& b) { return a <= b; });
  m.def("__gt__", [](const Tensor& a, const Tensor& b) { return a > b; });
  m.def("__ge__", [](const Tensor& a, const Tensor& b) { return a >= b; });
  m.def("__eq__", [](const Tensor& a, const Tensor& b) { return a == b; });
  m.def("LTFloat", [](const Tensor& a, float x) { return a < x; });
  m.def("LEFloat", [](const Tensor& a, float x) { return a <= x; });
  m.def("GTFloat", [](const Tensor& a, float x) { return a > x; });
  m.def("GEFloat", [](const Tensor& a, float x) { return a >= x; });
  m.def("EQFloat", [](const Tensor& a, float x) { return a == x; });

  m.def("ConcatOn", [](const std::vector<Tensor>& in, int axis) { return singa::ConcatOn(in, axis); });
  m.def("SliceOn", &singa::SliceOn);

  // arithmetic
  m.def("__add__", [](const Tensor& a, const Tensor& b) { return a + b; });
  m.def("__sub__", [](const Tensor& a, const Tensor& b) { return a - b; });
  m.def("__mul__", [](const Tensor& a, const Tensor& b) { return a * b; });
  m.def("__div__", [](const Tensor& a, const Tensor& b) { return a / b; });
  m.def("Add", static_cast<PairOut>(&singa::Add));
  m.def("Sub", static_cast<PairOut>(&singa::Sub));
  m.def("EltwiseMult", static_cast<PairOut>(&singa::EltwiseMult));
  m.def("Div", static_cast<PairOut>(&singa::Div));
  m.def("AddFloat", [](const Tensor& a, float x) { return a + x; });
  m.def("SubFloat", [](const Tensor& a, float x) { return a - x; });
  m.def("MultFloat", [](const Tensor& a, float x) { return a * x; });
  m.def("DivFloat", [](const Tensor& a, float x) { return a / x; });
  m.def("AddFloatWithRet", [](const Tensor& a, float x, Tensor* out) { singa::Add(a, x, out); });
  m.def("SubFloatWithRet", [](const Tensor& a, float x, Tensor* out) { singa::Sub(a, x, out); });
  m.def("EltwiseMultFloatWithRet", [](const Tensor& a, float x, Tensor* out) { singa::EltwiseMult(a, x, out); });
  m.def("DivFloatWithRet", [](const Tensor& a, float x, Tensor* out) { singa::Div(a, x, out); });

  // random
  m.def("Bernoulli", [](float p, Tensor* out) { singa::Bernoulli(p, out); });
  m.def("Gaussian", [](float mean, float std, Tensor* out) { singa::Gaussian(mean, std, out); });
  m.def("Uniform", [](float low, float high, Tensor* out) { singa::Uniform(low, high, out); });

  // BLAS
  m.def("Axpy", [](float alpha, const Tensor& in, Tensor* out) { singa::Axpy(alpha, in, out); });
  m.def("Axpy", [](const Tensor& alpha, const Tensor& in, Tensor* out) { singa::Axpy(alpha, in, out); });
  m.def("Mult", [](const Tensor& a, const Tensor& b) { return singa::Mult(a, b); });
  m.def("MultWithRet", [](const Tensor& a, const Tensor& b, Tensor* c) { singa::Mult(a, b, c); });
  m.def("MultWithScale",
        [](float alpha, const Tensor& a, const Tensor& b, float beta, Tensor* c) { singa::Mult(alpha, a, b, beta, c); });

  // matrix rows / columns
  m.def("AddColumn", static_cast<RowCol>(&singa::AddColumn));
  m.def("AddColumnWithScale",
        [](float alpha, float beta, const Tensor& v, Tensor* M) { singa::AddColumn(alpha, beta, v, M); });
  m.def("AddRow", static_cast<RowCol>(&singa::AddRow));
  m.def("AddRowWithScale", [](float alpha, float beta, const Tensor& v, Tensor* M) { singa::AddRow(alpha, beta, v, M); });
  m.def("DivColumn", &singa::DivColumn);
  m.def("DivRow", &singa::DivRow);
  m.def("MultColumn", &singa::MultColumn);
  m.def("MultRow", &singa::MultRow);
  m.def("SubColumn", &singa::SubColumn);
  m.def("SubRow", &singa::SubRow);
  m.def("SumColumns", &singa::SumColumns);
  m.def("SumRows", &singa::SumRows);

  m.def("CrossEntropyFwd", &singa::CrossEntropyFwd);
  m.def("SoftmaxCrossEntropyBwd", [](const Tensor& p, const Tensor& t) { return singa::SoftmaxCrossEntropyBwd(p, t); });
  m.def("InitLogging", [](const char* argv) { singa::InitLogging(argv); });
}
