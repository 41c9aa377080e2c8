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
import numpy as np
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
    sfx = _suffix(inp)
    assert out.dtype == inp.dtype
    if isinstance(alpha, torch.Tensor):
        _chk(alpha)
        alpha = alpha if alpha.dtype == _F32 else alpha.float()   # AsType(kFloat32), tensor_math_cuda.h:1056
        _lib.call("sgb_axpy_dev_alpha_" + sfx, _p(alpha), _p(inp), _p(out), inp.numel(), _stream())
    else:
        _lib.call("sgb_axpy_" + sfx, float(alpha), _p(inp), _p(out), inp.numel(), _stream())
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
    out = torch.empty(tuple(shape), dtype=t_storage.dtype, device=t_storage.device)
    sh = (C.c_int * len(shape))(*shape)
    st = (C.c_int * len(shape))(*stride)
    _lib.call("sgb_strided_copy_" + _suffix(t_storage), _p(t_storage), _p(out), n, len(shape),
              C.cast(sh, C.c_void_p), C.cast(st, C.c_void_p), _stream())
    return out


# ------------------------------------------------------------------ workspace
_WS = {}
_WS_RETIRED = []      # outgrown buffers: kept alive, never handed back to the allocator


def _workspace(device, nbytes):
    """A per-device scratch buffer owned by the host layer (the C ABI never
    allocates); 256-byte aligned by the torch allocator.  When a larger request
    arrives a new buffer takes over and the old one is RETIRED, not freed: its
    address may sit in a captured CUDA graph or in work queued on another
    stream, and must not be handed to someone else by the caching allocator.
    A graph captured through these wrappers therefore pins the workspace it saw.
    Growth during a stream capture is refused (it would allocate inside it)."""
    buf = _WS.get(device)
    if buf is None or buf.numel() < nbytes:
        if buf is not None and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("workspace of %d bytes needed during stream capture (have %d): run the call "
                               "once before capturing" % (nbytes, buf.numel()))
        if buf is not None:
            _WS_RETIRED.append(buf)
        buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _WS[device] = buf
    return buf


def _ws_args(device, nbytes):
    if nbytes == 0:
        return None, 0
    buf = _workspace(device, nbytes)
    return buf.data_ptr(), buf.numel()


# ------------------------------------------------------------------ reductions
def SumRows(M, v=None):
    """core_tensor.i:380 ``SumRows(M, v)``: v[c] = sum_r M[r, c]."""
    _chk(M)
    nrow, ncol = M.shape
    v = torch.empty(ncol, dtype=_F32, device=M.device) if v is None else v
    need = _lib.lib().sgb_sum_rows_workspace_bytes(nrow, ncol)
    ws, wsn = _ws_args(M.device, need)
    _lib.call("sgb_sum_rows_f32", _p(M), _p(v), nrow, ncol, ws, wsn, _stream())
    return v


def SumColumns(M, v=None):
    """core_tensor.i:379 ``SumColumns(M, v)``: v[r] = sum_c M[r, c]."""
    _chk(M)
    nrow, ncol = M.shape
    v = torch.empty(nrow, dtype=_F32, device=M.device) if v is None else v
    _lib.call("sgb_sum_columns_f32", _p(M), _p(v), nrow, ncol, _stream())
    return v


def Sum(t, axis):
    """core_tensor.i:223 ``Tensor Sum(t, axis)`` (tensor.cc:1229-1240)."""
    if axis == 0:
        return SumRows(t)
    assert axis == 1, "Not support Sum over axis = %d" % axis
    return SumColumns(t)


def SumAll(t):
    """core_tensor.i:226 ``Tensor SumAll(t)`` -> one-element device tensor."""
    _chk(t)
    out = torch.empty(1, dtype=_F32, device=t.device)
    need = _lib.lib().sgb_sum_all_workspace_bytes(t.numel())
    ws, wsn = _ws_args(t.device, need)
    _lib.call("sgb_sum_all_f32", _p(t), _p(out), t.numel(), ws, wsn, _stream())
    return out


def _blas1(fn, out_dtype, *tensors):
    _chk(*tensors)
    n = tensors[0].numel()
    out = torch.empty(1, dtype=out_dtype, device=tensors[0].device)
    ws, wsn = _ws_args(tensors[0].device, _lib.lib().sgb_blas1_workspace_bytes(n))
    _lib.call(fn, *([_p(t) for t in tensors] + [_p(out), n, ws, wsn, _stream()]))
    return out


def Dot(a, b):
    """Dot<float, lang::Cuda> (tensor_math_cuda.h:1084-1094, the Tensor*
    overload): one-element DEVICE tensor, no host synchronisation."""
    assert a.numel() == b.numel()
    return _blas1("sgb_dot_f32", _F32, a, b)


def Asum(t):
    """Asum<float, lang::Cuda> (tensor_math_cuda.h:1023-1029): sum of |x|."""
    return _blas1("sgb_asum_f32", _F32, t)


def Nrm2(t):
    """Nrm2<float, lang::Cuda> (tensor_math_cuda.h:1097-1102)."""
    return _blas1("sgb_nrm2_f32", _F32, t)


def Amax(t):
    """Amax<float, lang::Cuda> (tensor_math_cuda.h:1001-1009): 0-based index of
    the first element with the largest magnitude (int32 device tensor)."""
    return _blas1("sgb_amax_f32", _I32, t)


def Amin(t):
    """Amin<float, lang::Cuda> (tensor_math_cuda.h:1012-1020): smallest magnitude."""
    return _blas1("sgb_amin_f32", _I32, t)


def DGMM(side_right, M, v):
    """DGMM<float, lang::Cuda> (tensor_math_cuda.h:1112-1129): M * diag(v) when
    side_right else diag(v) * M, row-major M."""
    _chk(M, v)
    nrow, ncol = M.shape
    assert v.numel() == (ncol if side_right else nrow)
    out = torch.empty_like(M)
    _lib.call("sgb_dgmm_f32", int(bool(side_right)), _p(M), _p(v), _p(out), nrow, ncol, _stream())
    return out


def RowMax(t):
    _chk(t)
    v = torch.empty(t.shape[0], dtype=_F32, device=t.device)
    _lib.call("sgb_row_max_f32", _p(t), _p(v), t.shape[0], t.shape[1], _stream())
    return v


def GpuConvBackwardb(dy, b=None, cch=None):
    """model_operation.i:148: db[c] = sum_{n,h,w} dy (NCHW)."""
    _chk(dy)
    n, c = dy.shape[0], dy.shape[1]
    hw = dy.numel() // (n * c)
    db = torch.empty(c, dtype=_F32, device=dy.device)
    need = _lib.lib().sgb_conv_bias_backward_workspace_bytes(n, c, hw)
    ws, wsn = _ws_args(dy.device, need)
    _lib.call("sgb_conv_bias_backward_f32", _p(dy), _p(db), n, c, hw, ws, wsn, _stream())
    return db


# ------------------------------------------------------ softmax / cross entropy
def SoftMax(t, axis=None):
    """core_tensor.i:229-230.  ``axis`` reshapes to 2-D as tensor.cc:942-972
    does: rows = prod(shape[:axis]), columns = the rest."""
    _chk(t)
    if axis is None:
        nrow = t.shape[0] if t.dim() == 2 else 1
    else:
        axis = axis % t.dim()
        nrow = 1
        for s in t.shape[:axis]:
            nrow *= s
    y = torch.empty_like(t)
    _lib.call("sgb_softmax_rows_" + _suffix(t), _p(t), _p(y), nrow, t.numel() // max(nrow, 1), _stream())
    return y


def _ce_dims(p, t):
    batch = p.shape[0] if p.dim() == 2 else 1
    dim = p.numel() // batch
    assert t.dtype == _I32, "targets are int32 (kInt) tensors"
    return batch, dim, int(t.numel() == batch)


def CrossEntropyFwd(p, t):
    """core_tensor.i:387."""
    _chk(p, t)
    batch, dim, it = _ce_dims(p, t)
    loss = torch.empty(batch, dtype=p.dtype, device=p.device)
    _lib.call("sgb_cross_entropy_" + _suffix(p), it, batch, dim, _p(p), _p(t), _p(loss), _stream())
    return loss


def SoftmaxCrossEntropyBwd(p, t):
    """core_tensor.i:388: returns p - target in a new tensor."""
    _chk(p, t)
    batch, dim, it = _ce_dims(p, t)
    g = torch.empty_like(p)
    _lib.call("sgb_softmax_cross_entropy_bwd_" + _suffix(p), it, batch, dim, _p(p), _p(t), _p(g), _stream())
    return g


def SoftmaxCrossEntropyGrad(p, t, scale):
    """Fused SoftmaxCrossEntropyBwd + ``dx *= scale`` (autograd.py:1319-1322
    with scale = float32(1/N))."""
    _chk(p, t)
    batch, dim, it = _ce_dims(p, t)
    g = torch.empty_like(p)
    _lib.call("sgb_softmax_cross_entropy_grad_f32", it, batch, dim, _p(p), _p(t),
              float(scale), _p(g), _stream())
    return g


# ------------------------------------------------------------ operation handles
def SoftMaxCrossEntropyFused(logits, t, scale):
    """The loss head of autograd.SoftMaxCrossEntropy (python/singa/autograd.py:
    1306-1322) for integer targets in one launch.  Returns (prob, loss per
    sample, grad) with grad = (prob - onehot) * scale."""
    _chk(logits, t)
    assert t.dtype == _I32 and t.numel() == logits.shape[0], "one int32 target per sample"
    batch, dim = logits.shape
    prob, grad = torch.empty_like(logits), torch.empty_like(logits)
    loss = torch.empty(batch, dtype=_F32, device=logits.device)
    _lib.call("sgb_softmax_cross_entropy_fused_f32", _p(logits), _p(t), batch, dim, float(np.float32(scale)),
              _p(prob), _p(loss), _p(grad), _stream())
    return prob, loss, grad


class CudnnBatchNormHandle(object):
    """Shape record with the fields of singa's BatchNormHandle
    (src/model/operation/batchnorm.h:38-60); no cuDNN descriptors are needed."""

    def __init__(self, momentum, x):
        self.factor = momentum
        self.batchsize = x.shape[0]
        self.channels = x.shape[1]
        self.is_2d = x.dim() == 2
        self.height = 1 if self.is_2d else x.shape[2]
        self.width = 1 if self.is_2d else x.shape[3]


def GpuBatchNormForwardTraining(cbnh, x, bnScale, bnBias, running_mean, running_var, eps=0.0):
    """model_operation.i:159: returns [y, mean, var] where ``var`` is the saved
    INVERSE standard deviation 1/sqrt(batch_var + eps); running statistics are
    updated in place with ``cbnh.factor``.  ``eps`` defaults to the value the
    reference passes with cuDNN 9 (CUDNN_BN_MIN_EPSILON == 0)."""
    _chk(x, bnScale, bnBias, running_mean, running_var)
    n, c, hw = cbnh.batchsize, cbnh.channels, cbnh.height * cbnh.width
    y = torch.empty_like(x)
    mean = torch.empty_like(running_mean)
    var = torch.empty_like(running_var)
    need = _lib.lib().sgb_bn_backward_workspace_bytes(n, c, hw)
    ws, wsn = _ws_args(x.device, need)
    _lib.call("sgb_bn_forward_training_f32", _p(x), _p(bnScale), _p(bnBias), _p(running_mean),
              _p(running_var), float(cbnh.factor), float(eps), _p(y), _p(mean), _p(var), n, c, hw,
              ws, wsn, _stream())
    return [y, mean, var]


def GpuBatchNormBackward(cbnh, dy, x, bnScale, mean, var):
    """model_operation.i:165: returns [dx, dscale, dbias].  ``var`` is the
    saved INVERSE standard deviation produced by the forward pass, as in the
    reference (batchnorm.cc:314-321, 390-396)."""
    _chk(dy, x, bnScale, mean, var)
    n, c, hw = cbnh.batchsize, cbnh.channels, cbnh.height * cbnh.width
    dx = torch.empty_like(dy)
    ds = torch.empty_like(bnScale)
    db = torch.empty_like(bnScale)
    need = _lib.lib().sgb_bn_backward_workspace_bytes(n, c, hw)
    ws, wsn = _ws_args(dy.device, need)
    _lib.call("sgb_bn_backward_f32", _p(x), _p(dy), _p(bnScale), _p(mean), _p(var),
              _p(dx), _p(ds), _p(db), n, c, hw, ws, wsn, _stream())
    return [dx, ds, db]


def GpuBatchNormReLUBackward(cbnh, dy, relu_in, x, bnScale, mean, var):
    """ReLUBackward(dy, relu_in) followed by GpuBatchNormBackward, one pass."""
    _chk(dy, relu_in, x, bnScale, mean, var)
    n, c, hw = cbnh.batchsize, cbnh.channels, cbnh.height * cbnh.width
    dx = torch.empty_like(dy)
    ds = torch.empty_like(bnScale)
    db = torch.empty_like(bnScale)
    need = _lib.lib().sgb_bn_backward_workspace_bytes(n, c, hw)
    ws, wsn = _ws_args(dy.device, need)
    _lib.call("sgb_bn_relu_backward_f32", _p(x), _p(dy), _p(relu_in), _p(bnScale), _p(mean),
              _p(var), _p(dx), _p(ds), _p(db), n, c, hw, ws, wsn, _stream())
    return [dx, ds, db]


def GpuBatchNormAddReLUBackward(cbnh, dy_a, dy_b, relu_in, x, bnScale, mean, var):
    """The end of a residual block in one pass: the gradient join dy_a + dy_b
    (autograd.py:204 "+="), ReLUBackward against relu_in, GpuBatchNormBackward.
    Returns [joined, dx, dbnScale, dbnBias]; ``joined`` is what the shortcut
    branch consumes."""
    _chk(dy_a, dy_b, relu_in, x, bnScale, mean, var)
    n, c, hw = cbnh.batchsize, cbnh.channels, cbnh.height * cbnh.width
    joined = torch.empty_like(dy_a)
    dx = torch.empty_like(dy_a)
    ds = torch.empty_like(bnScale)
    db = torch.empty_like(bnScale)
    need = _lib.lib().sgb_bn_backward_workspace_bytes(n, c, hw)
    ws, wsn = _ws_args(dy_a.device, need)
    _lib.call("sgb_bn_add_relu_backward_f32", _p(x), _p(dy_a), _p(dy_b), _p(relu_in), _p(bnScale),
              _p(mean), _p(var), _p(joined), _p(dx), _p(ds), _p(db), n, c, hw, ws, wsn, _stream())
    return [joined, dx, ds, db]


class CudnnPoolingHandle(object):
    """Fields of singa's PoolingHandle (src/model/operation/pooling.h:41-78,
    pooling.cc:27-52)."""

    def __init__(self, x, kernel_size, stride, padding, is_max=True):
        self.kernel_h, self.kernel_w = kernel_size
        self.stride_h, self.stride_w = stride
        self.pad_h, self.pad_w = padding
        self.batchsize, self.channels, self.height, self.width = x.shape
        self.pooled_height = 1
        if self.stride_h > 0:
            self.pooled_height = (self.height + 2 * self.pad_h - self.kernel_h) // self.stride_h + 1
        self.pooled_width = (self.width + 2 * self.pad_w - self.kernel_w) // self.stride_w + 1
        self.is_max_pooling = is_max

    def _geom(self):
        return (self.batchsize, self.channels, self.height, self.width, self.kernel_h,
                self.kernel_w, self.pad_h, self.pad_w, self.stride_h, self.stride_w)


def GpuPoolingForward(cph, x):
    """model_operation.i:189."""
    _chk(x)
    y = torch.empty((cph.batchsize, cph.channels, cph.pooled_height, cph.pooled_width),
                    dtype=_F32, device=x.device)
    name = "sgb_maxpool_forward_f32" if cph.is_max_pooling else "sgb_avgpool_forward_f32"
    _lib.call(name, _p(x), _p(y), *cph._geom(), _stream())
    return y


def GpuPoolingBackward(cph, dy, x, y):
    """model_operation.i:191."""
    _chk(dy, x, y)
    dx = torch.empty_like(x)
    if cph.is_max_pooling:
        _lib.call("sgb_maxpool_backward_f32", _p(x), _p(y), _p(dy), _p(dx), *cph._geom(), _stream())
    else:
        _lib.call("sgb_avgpool_backward_f32", _p(dy), _p(dx), *cph._geom(), _stream())
    return dx


def GpuPoolingForwardArgmax(cph, x):
    """Max-pool forward that also returns the arg-max record (one uint8 per
    window: where its first maximum sits) for GpuPoolingBackwardArgmax."""
    _chk(x)
    assert cph.is_max_pooling
    shape = (cph.batchsize, cph.channels, cph.pooled_height, cph.pooled_width)
    y = torch.empty(shape, dtype=_F32, device=x.device)
    arg = torch.empty(shape, dtype=torch.uint8, device=x.device)
    _lib.call("sgb_maxpool_forward_argmax_f32", _p(x), _p(y), _p(arg), *cph._geom(), _stream())
    return y, arg


def GpuPoolingBackwardArgmax(cph, dy, argmax):
    """Max-pool backward from dy and the forward's arg-max record alone (no x,
    no y); equals GpuPoolingBackward bit for bit."""
    _chk(dy, argmax)
    dx = torch.empty((cph.batchsize, cph.channels, cph.height, cph.width), dtype=_F32, device=dy.device)
    _lib.call("sgb_maxpool_backward_argmax_f32", _p(dy), _p(argmax), _p(dx), *cph._geom(), _stream())
    return dx


# ------------------------------------------------------------- multi-tensor ops
def _ptr_table(tensors):
    import ctypes as C
    n = len(tensors)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in tensors])
    sizes = (C.c_size_t * n)(*[t.numel() for t in tensors])
    return ptrs, sizes, n


def sgd_update_multi(params, grads, moments, lr, momentum=0.0, dampening=0.0, weight_decay=0.0,
                     nesterov=False, grad_scale=1.0):
    """One launch group for SGD.apply over a list of parameter tensors."""
    _chk(*params)
    _chk(*grads)
    pp, sizes, n = _ptr_table(params)
    gp, _, _ = _ptr_table(grads)
    mp = None
    if momentum != 0:
        _chk(*moments)
        mp, _, _ = _ptr_table(moments)
    _lib.call("sgb_sgd_update_multi_f32", pp, gp, mp, sizes, n, float(lr), float(momentum),
              float(dampening), float(weight_decay), int(nesterov), float(grad_scale), _stream())


def pack(tensors, flat, offset=0):
    _chk(flat, *tensors)
    ptrs, sizes, n = _ptr_table(tensors)
    name = "sgb_pack_f32" if flat.dtype == _F32 else "sgb_pack_f32_to_f16"
    _lib.call(name, ptrs, sizes, n, _p(flat), offset, _stream())


def unpack(flat, tensors, offset=0, scale=1.0):
    _chk(flat, *tensors)
    ptrs, sizes, n = _ptr_table(tensors)
    name = "sgb_unpack_f32" if flat.dtype == _F32 else "sgb_unpack_f16_to_f32"
    _lib.call(name, _p(flat), offset, ptrs, sizes, n, float(scale), _stream())


# -------------------------------------------------------- sparsification kernels
def sparse_threshold(g, acc, thr):
    """s = g + acc, kept = |s| >= thr; returns (idx 1-based int32, val) of the
    kept non-zero entries in ascending order; ``acc`` (or None) is updated in
    place with the residual.  Synchronises to read the count."""
    _chk(g)
    n = g.numel()
    idx = torch.empty(max(n, 1), dtype=_I32, device=g.device)
    val = torch.empty(max(n, 1), dtype=_F32, device=g.device)
    nnz = torch.zeros(1, dtype=_I32, device=g.device)
    need = _lib.lib().sgb_sparse_workspace_bytes(n)
    ws, wsn = _ws_args(g.device, need)
    _lib.call("sgb_sparse_threshold_f32", _p(g), None if acc is None else _p(acc), n, float(thr),
              _p(idx), _p(val), _p(nnz), ws, wsn, _stream())
    k = int(nnz.item())
    return idx[:k], val[:k]


def sparse_topk(g, acc, k, mode="magnitude"):
    """The k entries of s = g + acc with the largest key (ties -> lower index),
    as (idx 1-based int32, val) in ascending index order; ``acc`` (or None)
    becomes s with the selected entries zeroed."""
    _chk(g)
    n = g.numel()
    k = min(int(k), n)
    idx = torch.empty(max(k, 1), dtype=_I32, device=g.device)
    val = torch.empty(max(k, 1), dtype=_F32, device=g.device)
    need = _lib.lib().sgb_sparse_workspace_bytes(n)
    ws, wsn = _ws_args(g.device, need)
    _lib.call("sgb_sparse_topk_f32", _p(g), None if acc is None else _p(acc), None, n, k,
              {"magnitude": 0, "compat": 1}[mode], _p(idx), _p(val), ws, wsn, _stream())
    return idx[:k], val[:k]


def topk_count(ratio, n):
    return int(_lib.lib().sgb_topk_count(float(ratio), int(n)))


def scatter_add(dst, idx, val):
    _chk(dst, idx, val)
    _lib.call("sgb_scatter_add_f32", _p(idx), _p(val), idx.numel(), None, _p(dst), dst.numel(),
              _stream())
    return dst
