"""Host-side mirror of the reference's ``singa_wrap`` names for the backward path.

The reference exposes its C++ tensor functions and operation handles to
Python through SWIG (src/api/core_tensor.i, src/api/model_operation.i).  This
module offers the same names, argument order and return conventions for the
functions on the backward path, over CUDA ``torch.Tensor`` storage (torch is
only the owner of device memory and streams here).  Every function calls the
C ABI in ``libsgb.so``; nothing is computed by torch and there is no CPU
path: a CPU tensor raises ``ValueError``.

Tensors must be contiguous, as ``singa::Tensor`` blocks are on this path.
"""
import torch

from . import _lib

_F32, _F16, _I32 = torch.float32, torch.float16, torch.int32


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _chk(*ts):
    for t in ts:
        if not t.is_cuda:
            raise ValueError("singa_b200 has no CPU path: tensor is on %s" % t.device)
        if not t.is_contiguous():
            raise ValueError("tensor must be contiguous")


def _p(t):
    return t.data_ptr()


def _suffix(t):
    if t.dtype == _F32:
        return "f32"
    if t.dtype == _F16:
        return "f16"
    raise TypeError("unsupported dtype %s" % t.dtype)


# ------------------------------------------------------------------ ReLU path
def ReLU(t):
    """core_tensor.i:203 ``Tensor ReLU(const Tensor&)``."""
    _chk(t)
    y = torch.empty_like(t)
    _lib.call("sgb_relu_" + _suffix(t), _p(t), _p(y), t.numel(), _stream())
    return y


def ReLUBackward(in1, in2):
    """core_tensor.i:221 ``Tensor ReLUBackward(in1 = dy, in2 = x)``."""
    _chk(in1, in2)
    assert in1.shape == in2.shape and in1.dtype == in2.dtype
    dx = torch.empty_like(in2)
    _lib.call("sgb_relu_backward_" + _suffix(in1), _p(in1), _p(in2), _p(dx),
              in1.numel(), _stream())
    return dx


def AddReLUBackward(dy_a, dy_b, x):
    """Fused ``(dy_a + dy_b)`` join followed by ReLUBackward (no reference
    counterpart as one call; equals ReLUBackward(dy_a + dy_b, x) bit for bit)."""
    _chk(dy_a, dy_b, x)
    dx = torch.empty_like(x)
    _lib.call("sgb_add_relu_backward_f32", _p(dy_a), _p(dy_b), _p(x), _p(dx),
              x.numel(), _stream())
    return dx


# ---------------------------------------------------------- elementwise family
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4,
          "gt": 5, "ge": 6, "eq": 7, "lt": 8, "le": 9}
SCALAR = {"add": 0, "mul": 1, "rdiv": 2, "pow": 3, "gt": 4, "ge": 5, "eq": 6,
          "lt": 7, "le": 8, "threshold": 9}
UNARY = {n: i for i, n in enumerate(
    ["abs", "sign", "exp", "erf", "ceil", "floor", "round", "rounde", "log",
     "sqrt", "square", "cos", "cosh", "acos", "acosh", "sin", "sinh", "asin",
     "asinh", "tan", "tanh", "atan", "atanh", "sigmoid", "softplus", "softsign"])}


def binary(op, a, b, out=None):
    """Tensor (op) tensor; ``out`` may alias an input (``a += b`` joins)."""
    _chk(a, b)
    assert a.shape == b.shape and a.dtype == b.dtype
    out = torch.empty_like(a) if out is None else out
    _lib.call("sgb_binary_" + _suffix(a), BINARY[op], _p(a), _p(b), _p(out),
              a.numel(), _stream())
    return out


def scalar(op, t, x, out=None):
    _chk(t)
    out = torch.empty_like(t) if out is None else out
    if t.dtype == _F16:
        assert op == "mul"
        _lib.call("sgb_scalar_mul_f16", _p(t), float(x), _p(out), t.numel(), _stream())
    else:
        _lib.call("sgb_scalar_f32", SCALAR[op], _p(t), float(x), _p(out), t.numel(), _stream())
    return out


def unary(op, t, out=None):
    _chk(t)
    out = torch.empty_like(t) if out is None else out
    _lib.call("sgb_unary_f32", UNARY[op], _p(t), _p(out), t.numel(), _stream())
    return out


def iAdd(t, other):
    """core_tensor.i:151 ``operator+=`` (the gradient join)."""
    return binary("add", t, other, out=t)


def EltwiseMultFloatWithRet(t, x, ret):
    """core_tensor.i:321-322."""
    return scalar("mul", t, x, out=ret)


def DivFloatWithRet(t, x, ret):
    """core_tensor.i:325-326: Div(t, x) is EltwiseMult(t, 1/x)
    (src/core/tensor/tensor_math.h:149-153)."""
    import numpy as np
    return scalar("mul", t, float(np.float32(1.0) / np.float32(x)), out=ret)


def Clamp(t, low, high, out=None):
    _chk(t)
    out = torch.empty_like(t) if out is None else out
    _lib.call("sgb_clamp_f32", float(low), float(high), _p(t), _p(out), t.numel(), _stream())
    return out


def SetValue(t, v):
    _chk(t)
    _lib.call("sgb_set_" + _suffix(t), float(v), _p(t), t.numel(), _stream())
    return t


def AsType(t, dtype):
    """core_tensor.i:129 ``Tensor::AsType`` for f32<->f16 and f32<->int."""
    _chk(t)
    out = torch.empty(t.shape, dtype=dtype, device=t.device)
    key = (t.dtype, dtype)
    names = {(_F32, _F16): "sgb_cast_f32_f16", (_F16, _F32): "sgb_cast_f16_f32",
             (_F32, _I32): "sgb_cast_f32_i32", (_I32, _F32): "sgb_cast_i32_f32"}
    if key not in names:
        raise TypeError("unsupported cast %s -> %s" % key)
    _lib.call(names[key], _p(t), _p(out), t.numel(), _stream())
    return out


def Axpy(alpha, inp, out):
    """core_tensor.i:345-347: ``out += alpha * in``; alpha is a python float
    or a one-element device tensor."""
    _chk(inp, out)
    if isinstance(alpha, torch.Tensor):
        _chk(alpha)
        _lib.call("sgb_axpy_dev_alpha_f32", _p(alpha), _p(inp), _p(out), inp.numel(), _stream())
    else:
        _lib.call("sgb_axpy_f32", float(alpha), _p(inp), _p(out), inp.numel(), _stream())
    return out


def Transform(t_storage, shape, stride):
    """Materialises a strided / broadcast view (element strides, 0 = broadcast)
    as a contiguous tensor: Transform<float, lang::Cuda>
    (src/core/tensor/tensor_math_cuda.h:238-298)."""
    import ctypes as C
    _chk(t_storage)
    n = 1
    for s in shape:
        n *= s
    out = torch.empty(tuple(shape), dtype=_F32, device=t_storage.device)
    sh = (C.c_int * len(shape))(*shape)
    st = (C.c_int * len(shape))(*stride)
    _lib.call("sgb_strided_copy_f32", _p(t_storage), _p(out), n, len(shape),
              C.cast(sh, C.c_void_p), C.cast(st, C.c_void_p), _stream())
    return out
