"""ctypes view of the two CUDA builds of apache/singa's core made by
``oracle/ref_cuda_build.py`` ("reference": its own CUDA back end; "sgb": this
repository's replacement back end on the same Tensor / Device sources), through
the doors of ``ref_cuda_doors.cc``.  TEST INFRASTRUCTURE ONLY.  Load ONE
variant per process: both define the same C++ symbols."""
import ctypes as C
import os

import numpy as np

from . import ref_cuda_build


class Core(object):
    def __init__(self, variant, device_id=0):
        import torch  # noqa: F401  (its CUDA libraries, NCCL included, are loaded first)
        path = ref_cuda_build.LIBS[variant]
        if not os.path.exists(path):
            raise ImportError("%s is not built" % path)
        if variant == "sgb":
            from singa_b200 import _lib
            _lib.lib()
        self.L = L = C.CDLL(path)
        self.variant = variant
        ptr_fns = ["rs_tensor_new", "rs_tensor_ptr", "rs_tensor_as_type", "rs_relu", "rs_relu_backward", "rs_add",
                   "rs_sub", "rs_eltwise_mult", "rs_div", "rs_sum_axis", "rs_sum_all", "rs_softmax",
                   "rs_cross_entropy_fwd", "rs_softmax_cross_entropy_bwd", "rs_mult", "rs_transpose", "rs_unary",
                   "rs_compare_scalar", "rs_row_max", "rs_bn_handle_new", "rs_pool_handle_new", "rs_pool_forward",
                   "rs_pool_backward", "rs_comm_new"]
        if variant == "sgb":
            ptr_fns.append("rs_conv_bias_backward")
        for f in ptr_fns:
            getattr(L, f).restype = C.c_void_p
        L.rs_tensor_size.restype = C.c_size_t
        L.rs_tensor_dim.restype = C.c_size_t
        L.rs_l1.restype = C.c_float
        L.rs_l2.restype = C.c_float
        L.rs_init(device_id)

    # ---- tensors
    def tensor(self, array):
        a = np.ascontiguousarray(array)
        dt = {np.dtype(np.float32): 0, np.dtype(np.int32): 2}[a.dtype]
        dims = (C.c_size_t * a.ndim)(*a.shape)
        h = C.c_void_p(self.L.rs_tensor_new(a.ndim, dims, dt))
        if dt == 0:
            self.L.rs_tensor_from_host_f32(h, a.ctypes.data_as(C.c_void_p))
        else:
            self.L.rs_tensor_from_host_i32(h, a.ctypes.data_as(C.c_void_p))
        return h

    def numpy(self, h):
        h = C.c_void_p(h) if not isinstance(h, C.c_void_p) else h
        nd = self.L.rs_tensor_ndim(h)
        shape = tuple(self.L.rs_tensor_dim(h, i) for i in range(nd))
        out = np.empty(shape, np.float32)
        self.L.rs_tensor_to_host_f32(h, out.ctypes.data_as(C.c_void_p))
        return out

    def call(self, name, *args):
        """Calls a door that returns a new tensor handle."""
        r = getattr(self.L, name)(*args)
        assert r, name
        return C.c_void_p(r)

    def free(self, h):
        self.L.rs_tensor_free(h)

    def three(self, name, *args):
        out = (C.c_void_p * 3)()
        getattr(self.L, name)(*args, out)
        return [C.c_void_p(v) for v in out]
