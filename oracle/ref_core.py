"""ctypes view of ``oracle/_ref/libref_core.so``: apache/singa's own lang::Cpp
core compiled by ``oracle/ref_core_build.py``.  TEST INFRASTRUCTURE ONLY (the
CPU comparator and the timed CPU baseline of benchmark configuration 1)."""
import ctypes as C
import os

import numpy as np

from . import ref_core_build

_lib = None


def available():
    return os.path.exists(ref_core_build.LIB)


def lib():
    global _lib
    if _lib is None:
        path = ref_core_build.build_ref_core()
        if path is None or not os.path.exists(path):
            raise ImportError("libref_core.so is not built and no reference tree is present")
        _lib = C.CDLL(path)
        _lib.refcore_mlp_create.restype = C.c_void_p
        _lib.refcore_mlp_step.restype = C.c_float
        _lib.refcore_mlp_hot_path_step.restype = C.c_float
        _lib.refcore_sum_all.restype = C.c_float
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f(a):
    return np.ascontiguousarray(a, np.float32)


class MLP(object):
    """The MLP of benchmark configuration 1 on singa::Tensor (lang::Cpp)."""

    def __init__(self, batch, dims, lr=0.05, momentum=0.9):
        self.batch, self.dims = int(batch), [int(d) for d in dims]
        arr = (C.c_int * len(self.dims))(*self.dims)
        self.h = C.c_void_p(lib().refcore_mlp_create(self.batch, arr, len(self.dims), C.c_float(lr),
                                                     C.c_float(momentum)))

    def close(self):
        if self.h:
            lib().refcore_mlp_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _shape(self, layer, which):
        return (self.dims[layer], self.dims[layer + 1]) if which in (0, 2) else (self.dims[layer + 1],)

    def set(self, layer, which, value):
        v = _f(value)
        assert v.shape == self._shape(layer, which)
        lib().refcore_mlp_set(self.h, layer, which, _p(v))

    def get(self, layer, which):
        out = np.empty(self._shape(layer, which), np.float32)
        lib().refcore_mlp_get(self.h, layer, which, _p(out))
        return out

    def step(self, x, labels, want_grads=False):
        x, labels = _f(x), np.ascontiguousarray(labels, np.int32)
        grads = None
        if want_grads:
            n = sum(self.dims[i] * self.dims[i + 1] + self.dims[i + 1] for i in range(len(self.dims) - 1))
            grads = np.empty(n, np.float32)
        loss = lib().refcore_mlp_step(self.h, _p(x), _p(labels), _p(grads) if want_grads else None)
        return float(loss), grads


def mlp_hot_path_step(mlp, logits, labels, relu_x, dgrad, wgrad):
    """Backward + update step without the contractions (see ref_core_doors.cc).
    relu_x / dgrad / wgrad: lists indexed by layer (dgrad[0] may be None)."""
    L = len(mlp.dims) - 1
    keep = []

    def table(arrs):
        out = (C.c_void_p * L)()
        for i in range(L):
            a = arrs[i] if i < len(arrs) else None
            if a is None:
                out[i] = None
            else:
                a = _f(a)
                keep.append(a)
                out[i] = a.ctypes.data
        return out
    lg, lab = _f(logits), np.ascontiguousarray(labels, np.int32)
    return float(lib().refcore_mlp_hot_path_step(mlp.h, _p(lg), _p(lab), table(relu_x), table(dgrad), table(wgrad)))


def relu_backward(dy, x):
    dy, x = _f(dy), _f(x)
    out = np.empty_like(dy)
    lib().refcore_relu_backward(_p(dy), _p(x), _p(out), C.c_size_t(dy.size))
    return out


def softmax(x):
    x = _f(x)
    out = np.empty_like(x)
    lib().refcore_softmax(_p(x), _p(out), C.c_size_t(x.shape[0]), C.c_size_t(x.shape[1]))
    return out


def cross_entropy(p, t):
    p, t = _f(p), np.ascontiguousarray(t, np.int32)
    out = np.empty(p.shape[0], np.float32)
    lib().refcore_cross_entropy(_p(p), _p(t), _p(out), C.c_size_t(p.shape[0]), C.c_size_t(p.shape[1]))
    return out


def softmax_cross_entropy_bwd(p, t):
    p, t = _f(p), np.ascontiguousarray(t, np.int32)
    out = np.empty_like(p)
    lib().refcore_softmax_cross_entropy_bwd(_p(p), _p(t), _p(out), C.c_size_t(p.shape[0]), C.c_size_t(p.shape[1]))
    return out


def sum_axis0(m):
    m = _f(m)
    out = np.empty(m.shape[1], np.float32)
    lib().refcore_sum_axis0(_p(m), _p(out), C.c_size_t(m.shape[0]), C.c_size_t(m.shape[1]))
    return out


def sum_all(x):
    x = _f(x).ravel()
    return float(lib().refcore_sum_all(_p(x), C.c_size_t(x.size)))


def sgd(param, grad, moment, lr, momentum, weight_decay):
    """In place on `param` and `moment` (float32 arrays)."""
    g = _f(grad)
    lib().refcore_sgd(_p(param), _p(g), _p(moment), C.c_size_t(param.size), C.c_float(lr), C.c_float(momentum),
                      C.c_float(weight_decay))
