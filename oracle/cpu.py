"""ctypes front end of ``oracle.c`` operating on numpy arrays.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Function names follow
the reference's operator names; every wrapper allocates its outputs and
returns them, leaving its inputs untouched unless stated.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path):
            path = _build.build_oracle()
        _lib = C.CDLL(path)
        _lib.orc_sum_all_f32.restype = C.c_float
        _lib.orc_sparse_threshold_f32.restype = C.c_size_t
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_pool_out.restype = C.c_int
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(n):
    lib().orc_set_num_threads(C.c_int(int(n)))


# ---------------------------------------------------------------- elementwise
def relu(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_relu_fwd_f32(C.c_size_t(x.size), _p(x), _p(y))
    return y


def relu_backward(dy, x):
    dy, x = _f32(dy), _f32(x)
    dx = np.empty_like(x)
    lib().orc_relu_bwd_f32(C.c_size_t(x.size), _p(dy), _p(x), _p(dx))
    return dx


def relu_backward_f16(dy, x):
    """Half-precision rule of the CUDA reference: the mask is ``x >= 0``
    (src/core/tensor/math_kernel.cu:261-271), unlike the fp32 kernel."""
    dy = np.asarray(dy, dtype=np.float16)
    x = np.asarray(x, dtype=np.float16)
    return np.where(x >= 0, dy, np.float16(0)).astype(np.float16)


def add_inplace(a, b):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    b = _f32(b)
    lib().orc_add_inplace_f32(C.c_size_t(a.size), _p(a), _p(b))
    return a


def scale_inplace(a, c):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().orc_scale_inplace_f32(C.c_size_t(a.size), _p(a), C.c_float(c))
    return a


# ------------------------------------------------------- softmax/cross-entropy
def softmax(x):
    x = _f32(x)
    y = np.empty_like(x)
    nrow = x.shape[0] if x.ndim == 2 else 1
    lib().orc_softmax_rows_f32(C.c_size_t(nrow), C.c_size_t(x.size // nrow),
                               _p(x), _p(y))
    return y


def cross_entropy_fwd(p, t):
    p, t = _f32(p), _i32(t)
    batch = p.shape[0] if p.ndim == 2 else 1
    dim = p.size // batch
    loss = np.empty(batch, np.float32)
    lib().orc_ce_fwd_f32(C.c_int(int(t.size == batch)), C.c_size_t(batch),
                         C.c_size_t(dim), _p(p), _p(t), _p(loss))
    return loss


def softmax_cross_entropy_bwd(p, t):
    p, t = _f32(p), _i32(t)
    batch = p.shape[0] if p.ndim == 2 else 1
    dim = p.size // batch
    g = np.empty_like(p)
    lib().orc_ce_bwd_f32(C.c_int(int(t.size == batch)), C.c_size_t(batch),
                         C.c_size_t(dim), _p(p), _p(t), _p(g))
    return g


# ------------------------------------------------------------------ reductions
def sum_rows(M):
    M = _f32(M)
    v = np.empty(M.shape[1], np.float32)
    lib().orc_sum_rows_f32(C.c_size_t(M.shape[0]), C.c_size_t(M.shape[1]),
                           _p(M), _p(v))
    return v


def sum_columns(M):
    M = _f32(M)
    v = np.empty(M.shape[0], np.float32)
    lib().orc_sum_columns_f32(C.c_size_t(M.shape[0]), C.c_size_t(M.shape[1]),
                              _p(M), _p(v))
    return v


def sum_all(x):
    x = _f32(x)
    return float(lib().orc_sum_all_f32(C.c_size_t(x.size), _p(x)))


def conv_bias_backward(dy):
    dy = _f32(dy)
    n, c = dy.shape[0], dy.shape[1]
    hw = dy.size // (n * c)
    db = np.empty(c, np.float32)
    lib().orc_conv_bias_bwd_f32(C.c_size_t(n), C.c_size_t(c), C.c_size_t(hw),
                                _p(dy), _p(db))
    return db


# ------------------------------------------------------------------ batch norm
def _nchw(x):
    n, c = x.shape[0], x.shape[1]
    return n, c, x.size // (n * c)


def bn_stats(x, eps=0.0):
    """Batch mean and saved inverse std of a (N,C,H,W) or (N,D) tensor."""
    x = _f32(x)
    n, c, hw = _nchw(x)
    mean = np.empty(c, np.float32)
    invstd = np.empty(c, np.float32)
    lib().orc_bn_stats_spatial_f32(C.c_size_t(n), C.c_size_t(c), C.c_size_t(hw),
                                   _p(x), C.c_double(eps), _p(mean), _p(invstd))
    return mean, invstd


def bn_backward(dy, x, scale, mean, invstd):
    """Returns (dx, dscale, dbias); (N,C,H,W) spatial or (N,D) per-activation."""
    x, dy = _f32(x), _f32(dy)
    scale, mean, invstd = _f32(scale).ravel(), _f32(mean).ravel(), _f32(invstd).ravel()
    n, c, hw = _nchw(x)
    dx = np.empty_like(x)
    ds = np.empty(c, np.float32)
    db = np.empty(c, np.float32)
    lib().orc_bn_bwd_spatial_f32(C.c_size_t(n), C.c_size_t(c), C.c_size_t(hw),
                                 _p(x), _p(dy), _p(scale), _p(mean), _p(invstd),
                                 _p(dx), _p(ds), _p(db))
    return dx, ds, db


# --------------------------------------------------------------------- pooling
def pool_out(size, k, pad, stride):
    return int(lib().orc_pool_out(C.c_int(size), C.c_int(k), C.c_int(pad),
                                  C.c_int(stride)))


def _pool_args(x, kernel, stride, pad):
    n, c, h, w = x.shape
    return [C.c_int(v) for v in (n, c, h, w, kernel[0], kernel[1], pad[0],
                                 pad[1], stride[0], stride[1])]


def _pool_shape(x, kernel, stride, pad):
    n, c, h, w = x.shape
    return (n, c, pool_out(h, kernel[0], pad[0], stride[0]),
            pool_out(w, kernel[1], pad[1], stride[1]))


def maxpool_forward(x, kernel, stride, pad, return_argmax=False):
    x = _f32(x)
    y = np.empty(_pool_shape(x, kernel, stride, pad), np.float32)
    am = np.empty(y.shape, np.int32)
    lib().orc_maxpool_fwd_f32(*_pool_args(x, kernel, stride, pad), _p(x), _p(y),
                              _p(am))
    return (y, am) if return_argmax else y


def maxpool_backward(dy, x, kernel, stride, pad):
    x, dy = _f32(x), _f32(dy)
    assert dy.shape == _pool_shape(x, kernel, stride, pad)
    dx = np.empty_like(x)
    lib().orc_maxpool_bwd_f32(*_pool_args(x, kernel, stride, pad), _p(x),
                              _p(dy), _p(dx))
    return dx


def avgpool_forward(x, kernel, stride, pad):
    x = _f32(x)
    y = np.empty(_pool_shape(x, kernel, stride, pad), np.float32)
    lib().orc_avgpool_fwd_f32(*_pool_args(x, kernel, stride, pad), _p(x), _p(y))
    return y


def avgpool_backward(dy, x_shape, kernel, stride, pad):
    dy = _f32(dy)
    dx = np.empty(tuple(x_shape), np.float32)
    assert dy.shape == _pool_shape(dx, kernel, stride, pad)
    lib().orc_avgpool_bwd_f32(*_pool_args(dx, kernel, stride, pad), _p(dy),
                              _p(dx))
    return dx


# ------------------------------------------------------------------------- SGD
def sgd_update(p, g, buf, lr, momentum=0.0, dampening=0.0, weight_decay=0.0,
               nesterov=False):
    """In place on p, g and buf (buf may be None when momentum == 0)."""
    for a in (p, g) + ((buf,) if buf is not None else ()):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    use_m = int(momentum != 0)
    lib().orc_sgd_update_f32(C.c_size_t(p.size), _p(p), _p(g),
                             _p(buf) if buf is not None else None,
                             C.c_float(lr), C.c_float(momentum),
                             C.c_float(dampening), C.c_float(weight_decay),
                             C.c_int(use_m), C.c_int(int(nesterov)))
    return p


# --------------------------------------------------------------- sparsification
def sparse_threshold(g, acc, thr):
    """Returns (idx 1-based int32, val, acc') following the intended semantics
    of src/io/communicator.cc:619-680; ``acc`` may be None."""
    g = _f32(g).ravel()
    acc2 = None if acc is None else _f32(acc).ravel().copy()
    idx = np.empty(g.size, np.int32)
    val = np.empty(g.size, np.float32)
    nnz = lib().orc_sparse_threshold_f32(C.c_size_t(g.size), _p(g),
                                         _p(acc2) if acc2 is not None else None,
                                         C.c_float(thr), _p(idx), _p(val))
    return idx[:nnz].copy(), val[:nnz].copy(), acc2


def scatter_add(dst, idx, val):
    assert dst.dtype == np.float32 and dst.flags.c_contiguous
    idx, val = _i32(idx), _f32(val)
    lib().orc_scatter_add_f32(C.c_size_t(idx.size), _p(idx), _p(val), _p(dst))
    return dst
