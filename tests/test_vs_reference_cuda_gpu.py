"""The new kernels against the reference's own CUDA path on the same device
buffers: its unmodified launchers (singa::cuda::*, compiled for sm_100a into
oracle/_ref/libref_cuda.so) and the cuDNN calls it issues for batch-norm and
pooling backward (oracle/_ref/libref_cudnn.so).  Skipped when those checker
libraries were not built (they need the reference tree at build time)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_CUDA = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
REF_CUDNN = os.path.join(ROOT, "oracle", "_ref", "libref_cudnn.so")


def p(t):
    return C.c_void_p(t.data_ptr())


@pytest.fixture(scope="module")
def sw():
    from singa_b200 import singa_wrap
    return singa_wrap


@pytest.fixture(scope="module")
def rc():
    if not os.path.exists(REF_CUDA):
        pytest.skip("oracle/_ref/libref_cuda.so not built")
    return C.CDLL(REF_CUDA)


@pytest.fixture(scope="module")
def rd():
    if not os.path.exists(REF_CUDNN):
        pytest.skip("oracle/_ref/libref_cudnn.so not built")
    try:
        lib = C.CDLL(REF_CUDNN)
    except OSError as e:
        pytest.skip("cuDNN not loadable: %s" % e)
    lib.refcudnn_bn_min_epsilon.restype = C.c_double
    return lib


def bits(t):
    return t.view(torch.int32 if t.element_size() == 4 else torch.int16)


@pytest.mark.parametrize("n", [1, 1023, 1000003, (1 << 22) + 1])
def test_elementwise_bit_identical_to_reference_kernels(sw, rc, n):
    g = torch.Generator(device="cuda").manual_seed(n)
    a = torch.randn(n, device="cuda", generator=g)
    b = torch.randn(n, device="cuda", generator=g)
    b[::7] = 0.0
    out = torch.empty(n, device="cuda")
    N = C.c_size_t(n)
    rc.ref_relubackward(N, p(a), p(b), p(out), None)
    assert torch.equal(bits(sw.ReLUBackward(a, b)), bits(out))
    rc.ref_relu(N, p(b), p(out), None)
    assert torch.equal(bits(sw.ReLU(b)), bits(out))
    for name, op in (("ref_add", "add"), ("ref_sub", "sub"), ("ref_mult", "mul"), ("ref_div", "div")):
        getattr(rc, name)(N, p(a), p(b + 3), p(out), None)
        assert torch.equal(bits(sw.binary(op, a, b + 3)), bits(out)), op
    rc.ref_mult_scalar(N, p(a), C.c_float(0.125), p(out), None)
    assert torch.equal(bits(sw.scalar("mul", a, 0.125)), bits(out))
    for name in ("exp", "log", "sqrt", "tanh", "sigmoid"):
        src = a.abs() + 1e-3 if name in ("log", "sqrt") else a
        getattr(rc, "ref_" + name)(N, p(src), p(out), None)
        assert torch.equal(bits(sw.unary(name, src)), bits(out)), name
    h = torch.empty(n, device="cuda", dtype=torch.float16)
    rc.ref_float2half(N, p(a * 100), p(h), None)
    assert torch.equal(bits(sw.AsType(a * 100, torch.float16)), bits(h))
    rc.ref_half2float(N, p(h), p(out), None)
    assert torch.equal(bits(sw.AsType(h, torch.float32)), bits(out))
    ha, hb, ho = a.half(), b.half(), torch.empty(n, device="cuda", dtype=torch.float16)
    rc.ref_relubackward_half(N, p(ha), p(hb), p(ho), None)
    assert torch.equal(bits(sw.ReLUBackward(ha, hb)), bits(ho))       # half rule: x >= 0 keeps dy
    from singa_b200 import _lib
    io = torch.empty(n, device="cuda", dtype=torch.int32)
    mine = torch.empty_like(io)
    s = torch.cuda.current_stream().cuda_stream
    sp = torch.empty(n, device="cuda")
    rc.ref_sparsabs(N, C.c_float(0.5), p(a), p(out), None)
    _lib.call("sgb_sparsabs_f32", 0.5, a.data_ptr(), sp.data_ptr(), n, s)
    assert torch.equal(bits(sp), bits(out))
    rc.ref_sparsindex(N, p(out), p(io), None)
    _lib.call("sgb_sparsindex_f32", out.data_ptr(), mine.data_ptr(), n, s)
    assert torch.equal(mine, io)
    rc.ref_generateindex(N, p(io), None)
    _lib.call("sgb_generateindex_i32", mine.data_ptr(), n, s)
    assert torch.equal(mine, io)
    torch.cuda.synchronize()


def test_cross_entropy_kernels_match_reference(sw, rc):
    g = torch.Generator(device="cuda").manual_seed(1)
    logits = torch.randn(32, 1000, device="cuda", generator=g) * 3
    prob = sw.SoftMax(logits)
    t = torch.randint(0, 1000, (32,), device="cuda", dtype=torch.int32, generator=g)
    loss = torch.empty(32, device="cuda")
    rc.ref_cross_entropy(1, C.c_size_t(32), C.c_size_t(1000), p(prob), p(t), p(loss), None)
    assert torch.equal(bits(sw.CrossEntropyFwd(prob, t)), bits(loss))
    grad = prob.clone()
    rc.ref_softmax_cross_entropy_bwd(1, C.c_size_t(32), C.c_size_t(1000), p(grad), p(t), p(grad), None)
    assert torch.equal(bits(sw.SoftmaxCrossEntropyBwd(prob, t)), bits(grad))
    ta = torch.randint(0, 3, (32, 1000), device="cuda", dtype=torch.int32, generator=g)
    ta[:, 0] += 1
    grad = prob.clone()
    rc.ref_softmax_cross_entropy_bwd(0, C.c_size_t(32), C.c_size_t(1000), p(grad), p(ta), p(grad), None)
    assert torch.equal(bits(sw.SoftmaxCrossEntropyBwd(prob, ta)), bits(grad))
    m = -torch.rand(37, 1000, device="cuda") - 1
    rm = torch.empty(37, device="cuda")
    rc.ref_row_max(C.c_size_t(37), C.c_size_t(1000), p(m), p(rm), None)
    assert torch.equal(sw.RowMax(m), rm)


@pytest.mark.parametrize("scale", [1e-3, 3.0])
def test_topk_index_set_equals_reference_sortbykey(sw, rc, scale):
    """The reference sorts all (value, index) pairs with a comparator that
    truncates both operands to int; the index SET of its first K entries is what
    the radix select returns in "compat" mode (ties -> lower index)."""
    n = 1000003
    g = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7)) * scale
    key, idx = g.clone(), torch.empty(n, dtype=torch.int32, device="cuda")
    rc.ref_generateindex(C.c_size_t(n), p(idx), None)
    rc.ref_sortbykey(C.c_size_t(n), p(key), p(idx), None)
    torch.cuda.synchronize()
    k = sw.topk_count(0.01, n)
    ref_set = torch.sort(idx[:k]).values
    mine, _ = sw.sparse_topk(g, None, k, "compat")
    assert torch.equal(mine, ref_set)
    if scale < 1:                       # every |g| < 1 ties at key 0: the first K indices win
        assert torch.equal(ref_set, torch.arange(1, k + 1, device="cuda", dtype=torch.int32))


@pytest.mark.parametrize("shape", [(32, 64, 56, 56), (32, 256, 14, 14), (8, 5, 7, 7), (32, 64, 112, 112),
                                   (16, 100, 1, 1)])
def test_batchnorm_backward_matches_cudnn_call(sw, rd, shape):
    N, Cc, H, W = shape
    is2d = int(H == 1 and W == 1)
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    x = torch.randn(shape, device="cuda", generator=g) * 1.5 + 0.2
    dy = torch.randn(shape, device="cuda", generator=g) * 1e-2
    sc = torch.rand(Cc, device="cuda", generator=g) + 0.5
    z, o = torch.zeros(Cc, device="cuda"), torch.ones(Cc, device="cuda")
    y, sm, si = torch.empty_like(x), torch.empty(Cc, device="cuda"), torch.empty(Cc, device="cuda")
    eps = C.c_double(rd.refcudnn_bn_min_epsilon())       # what the reference passes
    assert rd.refcudnn_bn_forward_training(is2d, N, Cc, H, W, eps, p(x), p(sc), p(z), p(y), p(z.clone()),
                                           p(o), C.c_double(0.1), p(sm), p(si), None) == 0
    dx, ds, db = torch.empty_like(x), torch.empty(Cc, device="cuda"), torch.empty(Cc, device="cuda")
    assert rd.refcudnn_bn_backward(is2d, N, Cc, H, W, eps, p(x), p(dy), p(sc), p(sm), p(si), p(dx), p(ds),
                                   p(db), None) == 0
    torch.cuda.synchronize()
    h = sw.CudnnBatchNormHandle(0.1, x.view(N, Cc) if is2d else x)
    # forward partner against cudnnBatchNormalizationForwardTraining (same factor, eps)
    rm2, rv2 = z.clone(), o.clone()
    my, mm, mv = sw.GpuBatchNormForwardTraining(h, x.view(N, Cc) if is2d else x, sc, z, rm2, rv2,
                                                eps=rd.refcudnn_bn_min_epsilon())
    rm_ref, rv_ref = z.clone(), o.clone()
    y2 = torch.empty_like(x)
    assert rd.refcudnn_bn_forward_training(is2d, N, Cc, H, W, eps, p(x), p(sc), p(z), p(y2), p(rm_ref),
                                           p(rv_ref), C.c_double(0.1), p(sm), p(si), None) == 0
    torch.cuda.synchronize()
    for name, a, b in (("y", my.view_as(x), y2), ("save_mean", mm, sm), ("save_invstd", mv, si),
                       ("running_mean", rm2, rm_ref), ("running_var", rv2, rv_ref)):
        rel = float((a - b).abs().max() / b.abs().max())
        assert rel <= 1e-5, (name, rel)
    mdx, mds, mdb = sw.GpuBatchNormBackward(h, dy, x, sc, sm, si)
    for name, a, b in (("dx", mdx, dx), ("dscale", mds, ds), ("dbias", mdb, db)):
        rel = float((a - b).abs().max() / b.abs().max())
        assert rel <= 1e-5, (name, rel)


POOL = [((64, 32, 24, 24), 2, 2, 0), ((64, 32, 8, 8), 2, 2, 0), ((8, 16, 112, 112), 3, 2, 1), ((4, 8, 9, 11), 3, 1, 1)]


@pytest.mark.parametrize("case", POOL)
def test_maxpool_backward_matches_cudnn_call(sw, rd, oracle, case):
    shape, k, s, pd = case
    N, Cc, H, W = shape
    OH, OW = (H + 2 * pd - k) // s + 1, (W + 2 * pd - k) // s + 1
    g = torch.Generator(device="cuda").manual_seed(k * 10 + s)
    x = torch.relu(torch.randn(shape, device="cuda", generator=g))       # many exact ties at 0
    dy = torch.randn(N, Cc, OH, OW, device="cuda", generator=g)
    y, dx = torch.empty(N, Cc, OH, OW, device="cuda"), torch.empty_like(x)
    args = (N, Cc, H, W, OH, OW, k, k, pd, pd, s, s)
    assert rd.refcudnn_pooling(0, 1, *args, p(x), p(y), None, None, None) == 0
    assert rd.refcudnn_pooling(1, 1, *args, p(x), p(y), p(dy), p(dx), None) == 0
    torch.cuda.synchronize()
    h = sw.CudnnPoolingHandle(x, (k, k), (s, s), (pd, pd), True)
    assert torch.equal(sw.GpuPoolingForward(h, x), y)
    mine = sw.GpuPoolingBackward(h, dy, x, y)
    if k <= s:
        assert torch.equal(bits(mine), bits(dx))         # one window per element: bit-identical
        return
    # Overlapping windows: the arg-max attribution is identical; cuDNN's
    # CUDNN_POOLING_MAX adds the contributions of an element that wins three or
    # more windows in a varying order, so only those sums may differ in the
    # last bits.
    _, am = oracle.maxpool_forward(x.cpu().numpy(), (k, k), (s, s), (pd, pd), return_argmax=True)
    wins = np.zeros((N, Cc, H * W), np.int32)
    for n in range(N):
        for c in range(Cc):
            np.add.at(wins[n, c], am[n, c].ravel(), 1)
    diff = (mine != dx).cpu().numpy().reshape(N, Cc, H * W)
    assert not (diff & (wins < 3)).any()
    assert float((mine - dx).abs().max()) <= 4e-6


def test_maxpool_tie_rule_first_maximum(sw, rd):
    x = torch.zeros(1, 1, 5, 5, device="cuda")
    dy = torch.arange(1, 10, device="cuda", dtype=torch.float32).view(1, 1, 3, 3)
    y, dx = torch.empty(1, 1, 3, 3, device="cuda"), torch.empty_like(x)
    args = (1, 1, 5, 5, 3, 3, 3, 3, 1, 1, 2, 2)
    rd.refcudnn_pooling(0, 1, *args, p(x), p(y), None, None, None)
    rd.refcudnn_pooling(1, 1, *args, p(x), p(y), p(dy), p(dx), None)
    torch.cuda.synchronize()
    h = sw.CudnnPoolingHandle(x, (3, 3), (2, 2), (1, 1), True)
    assert torch.equal(sw.GpuPoolingBackward(h, dy, x, y), dx)


@pytest.mark.parametrize("case", POOL)
def test_avgpool_matches_cudnn_call(sw, rd, case):
    shape, k, s, pd = case
    N, Cc, H, W = shape
    OH, OW = (H + 2 * pd - k) // s + 1, (W + 2 * pd - k) // s + 1
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(shape, device="cuda", generator=g)
    dy = torch.randn(N, Cc, OH, OW, device="cuda", generator=g)
    y, dx = torch.empty(N, Cc, OH, OW, device="cuda"), torch.empty_like(x)
    args = (N, Cc, H, W, OH, OW, k, k, pd, pd, s, s)
    assert rd.refcudnn_pooling(0, 0, *args, p(x), p(y), None, None, None) == 0
    assert rd.refcudnn_pooling(1, 0, *args, p(x), p(y), p(dy), p(dx), None) == 0
    torch.cuda.synchronize()
    h = sw.CudnnPoolingHandle(x, (k, k), (s, s), (pd, pd), False)
    assert float((sw.GpuPoolingForward(h, x) - y).abs().max() / y.abs().max()) <= 1e-5
    assert float((sw.GpuPoolingBackward(h, dy, x, y) - dx).abs().max() / dx.abs().max()) <= 1e-5


@pytest.mark.parametrize("shape", [(64, 32, 24, 24), (64, 32, 8, 8), (3, 5, 7, 3)])
def test_conv_bias_backward_matches_cudnn_call(sw, rd, shape):
    """GpuConvBackwardb's library call (cudnnConvolutionBackwardBias,
    convolution.cc:684-702) on the small CNN's two shapes and an odd one."""
    from singa_b200 import _lib
    L = _lib.lib()
    N, Cc, H, W = shape
    dy = torch.randn(shape, device="cuda")
    want, got = torch.empty(Cc, device="cuda"), torch.empty(Cc, device="cuda")
    assert rd.refcudnn_conv_bias_backward(N, Cc, H, W, p(dy), p(want), None) == 0
    ws = torch.empty(max(L.sgb_conv_bias_backward_workspace_bytes(N, Cc, H * W), 256), dtype=torch.uint8, device="cuda")
    _lib.call("sgb_conv_bias_backward_f32", dy.data_ptr(), got.data_ptr(), N, Cc, H * W, ws.data_ptr(), ws.numel(),
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    exact = dy.double().sum((0, 2, 3))
    scale = exact.abs().max().item()
    assert (got.double() - want.double()).abs().max().item() <= 1e-5 * scale
    assert (got.double() - exact).abs().max().item() <= 1e-5 * scale


def test_maxpool_forward_propagates_nan_like_cudnn(sw, rd):
    """The reference's pooling descriptor is built with CUDNN_PROPAGATE_NAN
    (pooling.h:90): a NaN anywhere in a window is the window's maximum."""
    from singa_b200 import _lib
    L = _lib.lib()
    for k, s, pd in ((3, 2, 1), (2, 2, 0)):
        N, Cc, H, W = 2, 3, 12, 12
        OH = (H + 2 * pd - k) // s + 1
        x = torch.randn(N, Cc, H, W, device="cuda")
        x[0, 0, 2, 2] = float("nan")
        x[1, 2, 7, 10] = float("nan")
        x[1, 1, 0, 0] = float("nan")
        want, got = torch.empty(N, Cc, OH, OH, device="cuda"), torch.empty(N, Cc, OH, OH, device="cuda")
        assert rd.refcudnn_pooling(0, 1, N, Cc, H, W, OH, OH, k, k, pd, pd, s, s, p(x), p(want), None, None, None) == 0
        _lib.call("sgb_maxpool_forward_f32", x.data_ptr(), got.data_ptr(), N, Cc, H, W, k, k, pd, pd, s, s,
                  torch.cuda.current_stream().cuda_stream)
        rec = torch.empty(N, Cc, OH, OH, dtype=torch.uint8, device="cuda")
        got2 = torch.empty_like(got)
        _lib.call("sgb_maxpool_forward_argmax_f32", x.data_ptr(), got2.data_ptr(), rec.data_ptr(), N, Cc, H, W, k, k,
                  pd, pd, s, s, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert torch.isnan(want).any()
        assert torch.equal(torch.isnan(got), torch.isnan(want))
        assert torch.equal(torch.isnan(got2), torch.isnan(want))
        keep = ~torch.isnan(want)
        assert torch.equal(got[keep], want[keep]) and torch.equal(got2[keep], want[keep])
        # backward: cuDNN sends a window's gradient to its first NaN; so do the kernel that
        # recomputes the winners from x and the one that reads the forward's record
        dy = torch.ones_like(want)
        dx_want, dx_got, dx_rec = torch.zeros_like(x), torch.zeros_like(x), torch.zeros_like(x)
        assert rd.refcudnn_pooling(1, 1, N, Cc, H, W, OH, OH, k, k, pd, pd, s, s, p(x), p(want), p(dy), p(dx_want),
                                   None) == 0
        _lib.call("sgb_maxpool_backward_f32", x.data_ptr(), got.data_ptr(), dy.data_ptr(), dx_got.data_ptr(), N, Cc, H,
                  W, k, k, pd, pd, s, s, torch.cuda.current_stream().cuda_stream)
        _lib.call("sgb_maxpool_backward_argmax_f32", dy.data_ptr(), rec.data_ptr(), dx_rec.data_ptr(), N, Cc, H, W, k,
                  k, pd, pd, s, s, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(dx_got, dx_want), "winners recomputed from x"
        assert torch.equal(dx_rec, dx_want), "winners from the forward's record"
