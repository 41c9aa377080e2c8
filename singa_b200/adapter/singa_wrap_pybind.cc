// `singa_wrap` as a pybind11 module: the names apache/singa's Python layer
// (python/singa/{tensor,autograd,layer,opt,device,model,utils}.py) takes from
// its SWIG-generated extension (interface files src/api/singa.i, config.i,
// core_tensor.i, core_device.i, model_operation.i, dist_communicator.i), bound
// to the same C++ classes and functions.  SWIG is not available where this is
// built; with this module in its place the reference's Python runs unchanged
// on a core library whose CUDA back end is this repository's.
//
// Conventions carried over from the SWIG interface:
//  * numpy typemaps: CopyFloatDataFromHostPtr(array) takes a 1-D float32 array,
//    GetFloatValue(n) returns one; likewise Int and HalfFloat;
//  * std::vector<Tensor> is the class VecTensor (append / len / iteration);
//  * operators are exposed under the names the Python layer calls
//    (__add__, AddFloat, LTFloat, iAddFloat through __iadd__, ...);
//  * std::shared_ptr<Device> is the holder of Device.
// Not bound: the convolution and RNN handles (the reference's convolution.cc
// and rnn.cc do not compile against cuDNN 9) and the Cpu* operations that need
// DNNL; the Python layer only touches them when such a layer is built.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <pybind11/stl_bind.h>

#include <memory>
#include <string>
#include <vector>

#include "singa/core/device.h"
#include "singa/core/tensor.h"
#include "singa/singa_config.h"
#include "singa/utils/logging.h"
#ifdef USE_CUDNN
#include "model/operation/batchnorm.h"
#include "model/operation/pooling.h"
#endif
#ifdef USE_DIST
#include "singa/io/communicator.h"
#endif

namespace py = pybind11;
using singa::Device;
using singa::Tensor;

PYBIND11_MAKE_OPAQUE(std::vector<singa::Tensor>);

namespace {

using FloatArray = py::array_t<float, py::array::c_style | py::array::forcecast>;
using IntArray = py::array_t<int, py::array::c_style | py::array::forcecast>;

template <typename T, typename Array>
void copy_from_host(const Tensor& t, const Array& a, size_t offset) {
  t.CopyDataFromHostPtr(reinterpret_cast<const T*>(a.data()), static_cast<size_t>(a.size()), offset);
}

template <typename T>
py::array_t<T> values(const Tensor& t, size_t num) {
  py::array_t<T> out(static_cast<py::ssize_t>(num));
  t.GetValue(out.mutable_data(), num);
  return out;
}

// In-place operators return the Python object they were called on.
template <typename F>
py::object inplace(py::object self, F f) {
  f(self.cast<Tensor&>());
  return self;
}

void bind_tensor(py::module_& m) {
  // data types are plain integers on the Python side (the Python layer keeps
  // them as dictionary keys and compares them with its own integer constants)
  m.attr("kFloat32") = static_cast<int>(singa::kFloat32);
  m.attr("kFloat16") = static_cast<int>(singa::kFloat16);
  m.attr("kInt") = static_cast<int>(singa::kInt);
  m.attr("kChar") = static_cast<int>(singa::kChar);
  m.attr("kDouble") = static_cast<int>(singa::kDouble);
  m.def("SizeOf", [](int t) { return singa::SizeOf(static_cast<singa::DataType>(t)); });
  m.def("Product", [](const std::vector<size_t>& s, int start, size_t len) { return singa::Product(s, start, len); },
        py::arg("shape"), py::arg("start") = 0, py::arg("len") = 0);

  py::class_<Tensor>(m, "Tensor")
      .def(py::init<>())
      .def(py::init([](const std::vector<size_t>& shape, int dtype) {
             return new Tensor(shape, static_cast<singa::DataType>(dtype));
           }),
           py::arg("shape"), py::arg("dtype") = 0)
      .def(py::init([](const std::vector<size_t>& shape, std::shared_ptr<Device> dev, int dtype) {
             return new Tensor(shape, dev, static_cast<singa::DataType>(dtype));
           }),
           py::arg("shape"), py::arg("dev"), py::arg("dtype") = 0)
      .def(py::init<const Tensor&>())
      .def("device", &Tensor::device)
      .def("GetFloatValue", [](const Tensor& t, size_t n) { return values<float>(t, n); })
      .def("GetIntValue", [](const Tensor& t, size_t n) { return values<int>(t, n); })
      .def("GetHalfFloatValue",
           [](const Tensor& t, size_t n) {
             py::array out(py::dtype("float16"), std::vector<py::ssize_t>{static_cast<py::ssize_t>(n)});
             t.get_value(reinterpret_cast<half_float::half*>(out.mutable_data()), n);
             return out;
           })
      .def("SetFloatValue", [](Tensor& t, float x) { t.SetValue(x); })
      .def("data_type", [](const Tensor& t) { return static_cast<int>(t.data_type()); })
      .def("shape", [](const Tensor& t) { return t.shape(); })
      .def("shape", [](const Tensor& t, size_t i) { return t.shape(i); })
      .def("transpose", [](const Tensor& t) { return t.transpose(); })
      .def("nDim", &Tensor::nDim)
      .def("initialized", &Tensor::initialized)
      .def("Size", &Tensor::Size)
      .def("MemSize", &Tensor::MemSize)
      .def("ResetLike", &Tensor::ResetLike)
      .def("AsType", [](Tensor& t, int d) { return t.AsType(static_cast<singa::DataType>(d)); })
      .def("ToType", [](Tensor& t, int d) { return t.ToType(static_cast<singa::DataType>(d)); })
      .def("ToDevice", [](Tensor& t, std::shared_ptr<Device> d) { t.ToDevice(d); })
      .def("ToHost", [](Tensor& t) { t.ToHost(); })
      .def("L2", &Tensor::L2)
      .def("L1", &Tensor::L1)
      .def("CopyFloatDataFromHostPtr",
           [](const Tensor& t, const FloatArray& a, size_t offset) { copy_from_host<float>(t, a, offset); },
           py::arg("src"), py::arg("offset") = 0)
      .def("CopyIntDataFromHostPtr",
           [](const Tensor& t, const IntArray& a, size_t offset) { copy_from_host<int>(t, a, offset); }, py::arg("src"),
           py::arg("offset") = 0)
      .def("CopyHalfFloatDataFromHostPtr",
           [](const Tensor& t, const py::array& a, size_t offset) {
             py::array h = py::array::ensure(a.attr("astype")("float16"), py::array::c_style);
             t.CopyDataFromHostPtr(reinterpret_cast<const half_float::half*>(h.data()), static_cast<size_t>(h.size()),
                                   offset);
           },
           py::arg("src"), py::arg("offset") = 0)
      .def("CopyData", &Tensor::CopyData)
      .def("RepeatData", &Tensor::RepeatData)
      .def("Clone", [](const Tensor& t) { return t.Clone(); })
      .def("Repeat", [](Tensor& t, std::vector<size_t> r, int axis) { return t.Repeat(r, axis); })
      .def("__iadd__", [](py::object s, const Tensor& o) { return inplace(s, [&](Tensor& t) { t += o; }); })
      .def("__isub__", [](py::object s, const Tensor& o) { return inplace(s, [&](Tensor& t) { t -= o; }); })
      .def("__imul__", [](py::object s, const Tensor& o) { return inplace(s, [&](Tensor& t) { t *= o; }); })
      .def("__itruediv__", [](py::object s, const Tensor& o) { return inplace(s, [&](Tensor& t) { t /= o; }); })
      .def("__idiv__", [](py::object s, const Tensor& o) { return inplace(s, [&](Tensor& t) { t /= o; }); })
      .def("__iadd__", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t += x; }); })
      .def("__isub__", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t -= x; }); })
      .def("__imul__", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t *= x; }); })
      .def("__itruediv__", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t /= x; }); })
      .def("__idiv__", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t /= x; }); })
      .def("iAddFloat", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t += x; }); })
      .def("iSubFloat", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t -= x; }); })
      .def("iMulFloat", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t *= x; }); })
      .def("iDivFloat", [](py::object s, float x) { return inplace(s, [&](Tensor& t) { t /= x; }); });

  // std::vector<Tensor> as the class VecTensor (bound by hand: Tensor's ==
  // returns a Tensor, which the generic vector binding cannot use)
  using Vec = std::vector<Tensor>;
  py::class_<Vec>(m, "VecTensor")
      .def(py::init<>())
      .def(py::init([](const py::iterable& items) {
        auto v = std::unique_ptr<Vec>(new Vec());
        for (py::handle h : items) v->push_back(h.cast<Tensor>());
        return v;
      }))
      .def("append", [](Vec& v, const Tensor& t) { v.push_back(t); })
      .def("push_back", [](Vec& v, const Tensor& t) { v.push_back(t); })
      .def("clear", [](Vec& v) { v.clear(); })
      .def("size", [](const Vec& v) { return v.size(); })
      .def("__len__", [](const Vec& v) { return v.size(); })
      .def("__getitem__",
           [](Vec& v, py::ssize_t i) -> Tensor& {
             if (i < 0) i += static_cast<py::ssize_t>(v.size());
             if (i < 0 || static_cast<size_t>(i) >= v.size()) throw py::index_error();
             return v[static_cast<size_t>(i)];
           },
           py::return_value_policy::reference_internal)
      .def("__iter__", [](Vec& v) { return py::make_iterator(v.begin(), v.end()); }, py::keep_alive<0, 1>());
}

void bind_device(py::module_& m) {
  py::class_<Device, std::shared_ptr<Device>>(m, "Device")
      .def("SetRandSeed", &Device::SetRandSeed)
      .def("host", &Device::host)
      .def("Reset", &Device::Reset)
      .def("id", &Device::id)
      .def("Sync", &Device::Sync)
      .def("ResetGraph", &Device::ResetGraph)
      .def("RunGraph", &Device::RunGraph, py::arg("serial") = false)
      .def("graph_enabled", &Device::graph_enabled)
      .def("EnableGraph", &Device::EnableGraph)
      .def("PrintTimeProfiling", &Device::PrintTimeProfiling)
      .def("SetVerbosity", &Device::SetVerbosity)
      .def("SetSkipIteration", &Device::SetSkipIteration)
      .def_static("EnableLazyAlloc", &Device::EnableLazyAlloc);

  py::class_<singa::Platform>(m, "Platform")
#ifdef USE_CUDA
      .def_static("GetNumGPUs", &singa::Platform::GetNumGPUs)
      .def_static("GetGPUIDs", &singa::Platform::GetGPUIDs)
      .def_static("GetGPUMemSize", [](int device) { return singa::Platform::GetGPUMemSize(device); })
      .def_static("DeviceQuery", &singa::Platform::DeviceQuery, py::arg("id"), py::arg("verbose") = false)
      .def_static("CreateCudaGPUs", &singa::Platform::CreateCudaGPUs, py::arg("num_devices"),
                  py::arg("init_size") = 0)
      .def_static("CreateCudaGPUsOn", &singa::Platform::CreateCudaGPUsOn, py::arg("devices"),
                  py::arg("init_size") = 0)
#endif
      .def_static("GetDefaultDevice", &singa::Platform::GetDefaultDevice);
}

}  // namespace

void bind_math(py::module_& m);        // singa_wrap_pybind_math.cc
void bind_operations(py::module_& m);  // singa_wrap_pybind_ops.cc

PYBIND11_MODULE(singa_wrap, m) {
  m.doc() = "apache/singa's singa_wrap interface over pybind11";
#ifdef USE_CUDA
  m.attr("USE_CUDA") = 1;
#else
  m.attr("USE_CUDA") = 0;
#endif
#ifdef USE_CUDNN
  m.attr("USE_CUDNN") = 1;
#else
  m.attr("USE_CUDNN") = 0;
#endif
#ifdef USE_DIST
  m.attr("USE_DIST") = 1;
#else
  m.attr("USE_DIST") = 0;
#endif
  m.attr("USE_OPENCL") = 0;
  m.attr("USE_DNNL") = 0;
  m.attr("USE_PYTHON") = 1;
  m.attr("USE_JAVA") = 0;
  m.attr("SINGA_MAJOR_VERSION") = SINGA_MAJOR_VERSION;
  m.attr("SINGA_MINOR_VERSION") = SINGA_MINOR_VERSION;
  m.attr("SINGA_PATCH_VERSION") = SINGA_PATCH_VERSION;
  m.attr("SINGA_VERSION") = SINGA_VERSION;
  bind_tensor(m);
  bind_device(m);
  bind_math(m);
  bind_operations(m);
}
