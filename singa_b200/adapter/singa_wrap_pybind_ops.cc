// singa_wrap (pybind11): the operation handles and Gpu* functions of
// src/api/model_operation.i that build against cuDNN 9 (batch normalisation
// and pooling), and the communicator of src/api/dist_communicator.i.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <pybind11/stl_bind.h>

#include <cstring>
#include <vector>

#include "singa/core/tensor.h"
#include "singa/singa_config.h"
#ifdef USE_CUDNN
#include "model/operation/batchnorm.h"
#include "model/operation/pooling.h"
#endif
#ifdef USE_DIST
#include "singa/io/communicator.h"
#endif

namespace py = pybind11;
using singa::Tensor;

PYBIND11_MAKE_OPAQUE(std::vector<singa::Tensor>);

void bind_operations(py::module_& m) {
#ifdef USE_CUDNN
  py::class_<singa::BatchNormHandle>(m, "BatchNormHandle")
      .def(py::init<const float, const Tensor&>())
      .def_readwrite("batchsize", &singa::BatchNormHandle::batchsize)
      .def_readwrite("factor", &singa::BatchNormHandle::factor);
  py::class_<singa::CudnnBatchNormHandle, singa::BatchNormHandle>(m, "CudnnBatchNormHandle")
      .def(py::init<const float, const Tensor&>());
  m.def("GpuBatchNormForwardTraining", &singa::GpuBatchNormForwardTraining);
  m.def("GpuBatchNormForwardInference", &singa::GpuBatchNormForwardInference);
  m.def("GpuBatchNormBackward", &singa::GpuBatchNormBackward);

  py::class_<singa::PoolingHandle>(m, "PoolingHandle")
      .def(py::init<const Tensor&, const std::vector<int>&, const std::vector<int>&, const std::vector<int>&,
                    const bool>(),
           py::arg("input"), py::arg("kernel_size"), py::arg("stride"), py::arg("padding"), py::arg("is_max") = true)
      .def_readwrite("batchsize", &singa::PoolingHandle::batchsize)
      .def_readwrite("stride_h", &singa::PoolingHandle::stride_h)
      .def_readwrite("stride_w", &singa::PoolingHandle::stride_w)
      .def_readwrite("kernel_h", &singa::PoolingHandle::kernel_h)
      .def_readwrite("kernel_w", &singa::PoolingHandle::kernel_w)
      .def_readwrite("pad_h", &singa::PoolingHandle::pad_h)
      .def_readwrite("pad_w", &singa::PoolingHandle::pad_w)
      .def_readwrite("pooled_height", &singa::PoolingHandle::pooled_height)
      .def_readwrite("pooled_width", &singa::PoolingHandle::pooled_width)
      .def_readwrite("is_max_pooling", &singa::PoolingHandle::is_max_pooling);
  py::class_<singa::CudnnPoolingHandle, singa::PoolingHandle>(m, "CudnnPoolingHandle")
      .def(py::init<const Tensor&, const std::vector<int>&, const std::vector<int>&, const std::vector<int>&,
                    const bool>(),
           py::arg("input"), py::arg("kernel_size"), py::arg("stride"), py::arg("padding"), py::arg("is_max") = true);
  m.def("GpuPoolingForward", &singa::GpuPoolingForward);
  m.def("GpuPoolingBackward", &singa::GpuPoolingBackward);
#endif  // USE_CUDNN

#ifdef USE_DIST
  py::class_<singa::NcclIdHolder>(m, "NcclIdHolder")
      .def(py::init<>())
      // the id as bytes, so that one process can create it and hand it to the others
      .def_property(
          "id_bytes",
          [](const singa::NcclIdHolder& h) { return py::bytes(reinterpret_cast<const char*>(&h.id), sizeof(h.id)); },
          [](singa::NcclIdHolder& h, const std::string& b) {
            if (b.size() != sizeof(h.id)) throw py::value_error("wrong size for an NCCL unique id");
            std::memcpy(&h.id, b.data(), sizeof(h.id));
          });
  py::class_<singa::Communicator>(m, "Communicator")
      .def(py::init<int>())
      .def(py::init<int, int, const singa::NcclIdHolder&, int>())
      .def_readwrite("global_rank", &singa::Communicator::global_rank)
      .def_readwrite("world_size", &singa::Communicator::world_size)
      .def_readwrite("local_rank", &singa::Communicator::local_rank)
      .def("synch", &singa::Communicator::synch)
      .def("fusedSynch", &singa::Communicator::fusedSynch, py::arg("t"), py::arg("send") = true)
      .def("synchHalf", &singa::Communicator::synchHalf)
      .def("fusedSynchHalf", &singa::Communicator::fusedSynchHalf, py::arg("t"), py::arg("send") = true)
      .def("sparsification", [](singa::Communicator& c, Tensor& t, Tensor& acc, float s, bool topk) {
        c.sparsification(t, acc, s, topk);
      })
      .def("sparsification", [](singa::Communicator& c, Tensor& t, float s, bool topk) { c.sparsification(t, s, topk); })
      .def("fusedSparsification", [](singa::Communicator& c, std::vector<Tensor>& t, Tensor& acc, float s, bool topk) {
        c.fusedSparsification(t, acc, s, topk);
      })
      .def("fusedSparsification",
           [](singa::Communicator& c, std::vector<Tensor>& t, float s, bool topk) { c.fusedSparsification(t, s, topk); })
      .def("wait", &singa::Communicator::wait);
#endif  // USE_DIST
}
