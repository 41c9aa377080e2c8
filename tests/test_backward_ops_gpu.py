"""GPU parity of the reductions, softmax-cross-entropy, batch-norm and pooling
backward, the fused SGD update and bucket pack/unpack against the CPU oracle
and the reference's golden vectors.  All calls go through the C ABI.

Tolerances (stated by the task for this path): bit-exact for ReLU / pooling
arg-max gradients and pack/unpack; 1e-5 relative (to the largest expected
magnitude of the tensor) for fp32 reductions; 1e-3 for fp16."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL32 = 1e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def close(got, want, rtol=RTOL32, what=""):
    want = np.asarray(want, np.float64)
    got = np.asarray(got, np.float64)
    scale = max(np.abs(want).max() if want.size else 0.0, 1e-30)
    err = np.abs(got - want).max() if want.size else 0.0
    assert err <= rtol * scale, "%s: max err %.3e vs scale %.3e (rel %.2e)" % (what, err, scale, err / scale)


@pytest.fixture(scope="module")
def sw():
    from singa_b200 import singa_wrap
    return singa_wrap


# ------------------------------------------------------------------ reductions
@pytest.mark.parametrize("shape", [(1, 1), (3, 2), (256, 10), (256, 4096), (32, 1000), (64, 500),
                                   (5000, 33), (70000, 7), (2, 100003)])
def test_sum_rows_columns(sw, oracle, shape):
    rng = np.random.default_rng(shape[0] * 131 + shape[1])
    m = rng.standard_normal(shape).astype(np.float32)
    close(host(sw.SumRows(dev(m))), oracle.sum_rows(m), what="SumRows")
    close(host(sw.SumColumns(dev(m))), oracle.sum_columns(m), what="SumColumns")
    close(host(sw.Sum(dev(m), 0)), m.astype(np.float64).sum(0), what="Sum axis 0")


def test_sum_all_row_max_conv_bias(sw, oracle):
    rng = np.random.default_rng(3)
    for n in (1, 255, 256, 100003, 1 << 22):
        x = rng.standard_normal(n).astype(np.float32) + 0.5
        close(host(sw.SumAll(dev(x))), [oracle.sum_all(x)], what="SumAll %d" % n)
    m = -np.abs(rng.standard_normal((37, 1000)).astype(np.float32)) - 1.0   # all-negative rows
    assert np.array_equal(host(sw.RowMax(dev(m))), m.max(axis=1))
    for shape in [(64, 32, 24, 24), (64, 32, 8, 8), (3, 5, 7, 7), (2, 3, 1, 1), (32, 2048, 7, 7)]:
        dy = rng.standard_normal(shape).astype(np.float32)
        close(host(sw.GpuConvBackwardb(dev(dy))), oracle.conv_bias_backward(dy), what="conv bias %s" % (shape,))


# ------------------------------------------------------ softmax / cross entropy
def test_cross_entropy_golden(sw, golden):
    g = golden["cross_entropy"]
    logits = np.array(g["logits"], np.float32).reshape(g["shape"])
    p = sw.SoftMax(dev(logits))
    np.testing.assert_allclose(host(p), 0.25, rtol=1e-6)
    want = np.float32(-np.log(0.25))
    for t in (np.array(g["int_target"], np.int32), np.array(g["array_target"], np.int32).reshape(g["shape"])):
        np.testing.assert_allclose(host(sw.CrossEntropyFwd(p, dev(t))), want, rtol=1e-6)
        np.testing.assert_allclose(host(sw.SoftmaxCrossEntropyBwd(p, dev(t))).ravel(), g["grad"], rtol=1e-6)


@pytest.mark.parametrize("shape", [(256, 10), (64, 10), (32, 1000), (1, 7), (5, 4099)])
def test_softmax_cross_entropy_random(sw, oracle, shape):
    rng = np.random.default_rng(shape[1])
    logits = (rng.standard_normal(shape) * 3).astype(np.float32)
    logits[0] -= 50.0                       # an all-negative row
    t = rng.integers(0, shape[1], shape[0]).astype(np.int32)
    p_ref = oracle.softmax(logits)
    p = sw.SoftMax(dev(logits))
    close(host(p), p_ref, rtol=1e-5, what="softmax")
    np.testing.assert_allclose(host(p).sum(axis=1), 1.0, rtol=1e-5)
    # downstream ops are checked on the oracle's probabilities: bit-exact
    pd = dev(p_ref)
    loss = host(sw.CrossEntropyFwd(pd, dev(t)))
    np.testing.assert_allclose(loss, oracle.cross_entropy_fwd(p_ref, t), rtol=2e-6)
    g = host(sw.SoftmaxCrossEntropyBwd(pd, dev(t)))
    assert np.array_equal(g, oracle.softmax_cross_entropy_bwd(p_ref, t))
    inv = np.float32(1.0) / np.float32(shape[0])
    gs = host(sw.SoftmaxCrossEntropyGrad(pd, dev(t), float(inv)))
    assert np.array_equal(gs, oracle.softmax_cross_entropy_bwd(p_ref, t) * inv)
    ta = rng.integers(0, 3, shape).astype(np.int32)
    ta[:, 0] += 1
    g = host(sw.SoftmaxCrossEntropyBwd(pd, dev(ta)))
    np.testing.assert_allclose(g, oracle.softmax_cross_entropy_bwd(p_ref, ta), rtol=1e-6, atol=1e-7)
    close(host(sw.SumAll(sw.CrossEntropyFwd(pd, dev(t)))), [oracle.sum_all(oracle.cross_entropy_fwd(p_ref, t))],
          what="loss sum")


@pytest.mark.parametrize("shape", [(256, 10), (64, 10), (32, 1000), (1, 7), (5, 4099)])
def test_fused_loss_head_equals_the_three_kernels(sw, shape):
    rng = np.random.default_rng(shape[1] + 1)
    logits = dev((rng.standard_normal(shape) * 3).astype(np.float32))
    t = dev(rng.integers(0, shape[1], shape[0]).astype(np.int32))
    inv = float(np.float32(1.0) / np.float32(shape[0]))
    p = sw.SoftMax(logits)
    loss = sw.CrossEntropyFwd(p, t)
    grad = sw.SoftmaxCrossEntropyGrad(p, t, inv)
    fp, fl, fg = sw.SoftMaxCrossEntropyFused(logits, t, inv)
    assert torch.equal(fp, p) and torch.equal(fl, loss) and torch.equal(fg, grad)


# ------------------------------------------------------------------ batch norm
def bn_case(rng, shape):
    x = (rng.standard_normal(shape) * 1.7 + 0.3).astype(np.float32)
    dy = (rng.standard_normal(shape) * 1e-2).astype(np.float32)
    c = shape[1]
    scale = (rng.random(c) + 0.5).astype(np.float32)
    return x, dy, scale


def test_batchnorm_golden(sw, oracle, golden):
    g = golden["batchnorm"]
    x = np.array(g["bwd_x"], np.float32).reshape(g["shape"])
    dy = np.array(g["bwd_dy"], np.float32).reshape(g["shape"])
    mean, invstd = oracle.bn_stats(x, eps=g["eps"])
    h = sw.CudnnBatchNormHandle(0.9, dev(x))
    dx, ds, db = sw.GpuBatchNormBackward(h, dev(dy), dev(x), dev(np.array(g["bwd_scale"], np.float32)),
                                         dev(mean), dev(invstd))
    np.testing.assert_allclose(host(dx).ravel(), g["dx"], atol=g["tol"])
    np.testing.assert_allclose(host(ds), g["dscale"], atol=g["tol"])
    np.testing.assert_allclose(host(db), g["dbias"], atol=g["tol"])
    g = golden["batchnorm_api"]
    x = np.array(g["x"], np.float32).reshape(g["shape"])
    mean, invstd = oracle.bn_stats(x, eps=g["eps"])
    h = sw.CudnnBatchNormHandle(0.9, dev(x))
    dx = sw.GpuBatchNormBackward(h, dev(x), dev(x), dev(np.array(g["scale"], np.float32)), dev(mean), dev(invstd))[0]
    np.testing.assert_array_almost_equal(host(dx), np.array(g["dx"], np.float32), decimal=g["decimal"])


def _bn_training_model(x, scale, bias, rm, rv, momentum, e=1e-5):
    """The numpy statement of training-mode batch norm that the reference's API
    test checks cuDNN against (test/python/test_api.py:31-54), in float64."""
    x = x.astype(np.float64)
    axes = (0, 2, 3)
    bm, bv = x.mean(axis=axes), x.var(axis=axes)
    shape = (1, -1, 1, 1)
    y = (x - bm.reshape(shape)) / np.sqrt(bv.reshape(shape) + e) * scale.reshape(shape) + bias.reshape(shape)
    m = x.size // x.shape[1]
    return (y, momentum * bm + (1 - momentum) * rm, momentum * bv * m / (m - 1) + (1 - momentum) * rv, bm,
            1.0 / np.sqrt(bv))


def test_batchnorm_training_api_golden(sw, oracle, golden):
    g = golden["batchnorm_training_api"]
    dec = g["decimals"]
    cases = [(np.array(g["x"], np.float32).reshape(g["x_shape"]), np.array(g["scale"], np.float32),
              np.array(g["bias"], np.float32), np.array(g["running_mean"], np.float32),
              np.array(g["running_var"], np.float32), m) for m in g["momenta"]]
    rng = np.random.default_rng(0)
    shp = g["random_case"]["shape"]
    cases.append((rng.random(shp, dtype=np.float32),) + tuple(rng.random(shp[1], dtype=np.float32) for _ in range(4))
                 + (g["random_case"]["momentum"],))
    for x, s0, b0, rm0, rv0, mom in cases:
        y1, rm1, rv1, bm1, bv1 = _bn_training_model(x, s0, b0, rm0, rv0, mom)
        h = sw.CudnnBatchNormHandle(mom, dev(x))
        rm, rv = dev(rm0), dev(rv0)
        y, bm, bv = sw.GpuBatchNormForwardTraining(h, dev(x), dev(s0), dev(b0), rm, rv)
        np.testing.assert_array_almost_equal(host(y), y1, decimal=dec["y"])
        np.testing.assert_array_almost_equal(host(bm), bm1, decimal=dec["batch_mean"])
        np.testing.assert_array_almost_equal(host(rm), rm1, decimal=dec["running_mean"] - 1)
        np.testing.assert_array_almost_equal(host(bv), bv1, decimal=dec["saved_inv_std"])
        np.testing.assert_array_almost_equal(host(rv), rv1, decimal=dec["running_var"])
        om, oi = oracle.bn_stats(x)
        np.testing.assert_array_almost_equal(om, bm1, decimal=dec["batch_mean"])
        np.testing.assert_array_almost_equal(oi, bv1, decimal=dec["saved_inv_std"])


BN_SHAPES = [(1, 1, 1, 1), (2, 3, 4, 4), (4, 5, 7, 7), (3, 2, 5, 3), (8, 16, 14, 14), (32, 64, 28, 28),
             (32, 2048, 7, 7), (32, 64, 56, 56), (16, 100), (256, 4096), (7, 3),
             (3, 8, 5, 5), (2, 6, 3, 2), (32, 512, 7, 7), (5, 12, 3, 3), (32, 256, 56, 56)]


@pytest.mark.parametrize("shape", BN_SHAPES)
def test_batchnorm_forward_training(sw, oracle, shape):
    rng = np.random.default_rng(sum(shape) + 7)
    x, _, scale = bn_case(rng, shape)
    c = shape[1]
    bias = rng.standard_normal(c).astype(np.float32)
    rm0, rv0 = rng.standard_normal(c).astype(np.float32), (rng.random(c) + 0.5).astype(np.float32)
    eps = 1e-5
    mean, invstd = oracle.bn_stats(x, eps=eps)
    h = sw.CudnnBatchNormHandle(0.1, dev(x))
    rm, rv = dev(rm0), dev(rv0)
    y, m, v = sw.GpuBatchNormForwardTraining(h, dev(x), dev(scale), dev(bias), rm, rv, eps=eps)
    close(host(m), mean, what="mean %s" % (shape,))
    close(host(v), invstd, what="invstd %s" % (shape,))
    bshape = (1, c) + (1,) * (x.ndim - 2)
    want = (x.astype(np.float64) - mean.reshape(bshape)) * invstd.reshape(bshape) * scale.reshape(bshape) \
        + bias.reshape(bshape)
    close(host(y), want, rtol=2e-5, what="y %s" % (shape,))
    axes = (0,) + tuple(range(2, x.ndim))
    M = x.size // c
    var_unbiased = x.astype(np.float64).var(axis=axes) * (M / (M - 1.0) if M > 1 else 1.0)
    close(host(rm), 0.9 * rm0 + 0.1 * x.astype(np.float64).mean(axis=axes), what="running mean")
    close(host(rv), 0.9 * rv0 + 0.1 * var_unbiased, what="running var")


@pytest.mark.parametrize("shape", BN_SHAPES)
def test_batchnorm_backward(sw, oracle, shape):
    rng = np.random.default_rng(sum(shape))
    x, dy, scale = bn_case(rng, shape)
    mean, invstd = oracle.bn_stats(x, eps=0.0 if x.size > shape[1] else 1e-5)
    if not np.isfinite(invstd).all():
        invstd = np.ones_like(invstd)
    want = oracle.bn_backward(dy, x, scale, mean, invstd)
    h = sw.CudnnBatchNormHandle(0.9, dev(x))
    got = sw.GpuBatchNormBackward(h, dev(dy), dev(x), dev(scale), dev(mean), dev(invstd))
    for name, a, b in zip(("dx", "dscale", "dbias"), got, want):
        close(host(a), b, what="%s %s" % (name, shape))


@pytest.mark.parametrize("shape", [(2, 3, 4, 4), (4, 5, 7, 7), (8, 16, 14, 14), (32, 64, 28, 28), (32, 64, 7, 7),
                                   (2, 6, 3, 2), (32, 128, 56, 56)])
def test_batchnorm_relu_fused_equals_unfused(sw, oracle, shape):
    rng = np.random.default_rng(sum(shape) + 1)
    x, dy, scale = bn_case(rng, shape)
    relu_in = rng.standard_normal(shape).astype(np.float32)
    relu_in[0, 0].flat[0] = 0.0
    mean, invstd = oracle.bn_stats(x)
    h = sw.CudnnBatchNormHandle(0.9, dev(x))
    masked = sw.ReLUBackward(dev(dy), dev(relu_in))
    unfused = sw.GpuBatchNormBackward(h, masked, dev(x), dev(scale), dev(mean), dev(invstd))
    fused = sw.GpuBatchNormReLUBackward(h, dev(dy), dev(relu_in), dev(x), dev(scale), dev(mean), dev(invstd))
    for a, b in zip(fused, unfused):
        assert torch.equal(a, b)
    want = oracle.bn_backward(oracle.relu_backward(dy, relu_in), x, scale, mean, invstd)
    for a, b in zip(fused, want):
        close(host(a), b, what="fused bn+relu %s" % (shape,))


@pytest.mark.parametrize("shape", [(2, 3, 4, 4), (4, 5, 7, 7), (8, 16, 14, 14), (32, 64, 28, 28), (32, 64, 7, 7),
                                   (2, 6, 3, 2), (32, 256, 56, 56), (32, 64, 112, 112)])
def test_batchnorm_join_relu_fused_equals_unfused(sw, oracle, shape):
    rng = np.random.default_rng(sum(shape) + 2)
    x, dy_a, scale = bn_case(rng, shape)
    dy_b = rng.standard_normal(shape).astype(np.float32) * np.float32(1e-2)
    relu_in = rng.standard_normal(shape).astype(np.float32)
    relu_in[0, 0].flat[0] = 0.0
    mean, invstd = oracle.bn_stats(x)
    h = sw.CudnnBatchNormHandle(0.9, dev(x))
    joined = sw.AddReLUBackward(dev(dy_a), dev(dy_b), dev(relu_in))
    unfused = sw.GpuBatchNormBackward(h, joined, dev(x), dev(scale), dev(mean), dev(invstd))
    fused = sw.GpuBatchNormAddReLUBackward(h, dev(dy_a), dev(dy_b), dev(relu_in), dev(x), dev(scale), dev(mean),
                                           dev(invstd))
    for a, b in zip(fused, [joined] + unfused):
        assert torch.equal(a, b)
    want_joined = oracle.relu_backward(dy_a + dy_b, relu_in)
    assert np.array_equal(host(fused[0]), want_joined)
    want = oracle.bn_backward(want_joined, x, scale, mean, invstd)
    for a, b in zip(fused[1:], want):
        close(host(a), b, what="fused join+relu+bn %s" % (shape,))


def test_batchnorm_backward_resnet_stem_size(sw, oracle):
    shape = (32, 64, 112, 112)
    rng = np.random.default_rng(11)
    x = rng.standard_normal(shape, dtype=np.float32)
    dy = rng.standard_normal(shape, dtype=np.float32) * np.float32(1e-2)
    scale = np.ones(64, np.float32)
    mean, invstd = oracle.bn_stats(x)
    want = oracle.bn_backward(dy, x, scale, mean, invstd)
    h = sw.CudnnBatchNormHandle(0.9, dev(x))
    got = sw.GpuBatchNormBackward(h, dev(dy), dev(x), dev(scale), dev(mean), dev(invstd))
    for name, a, b in zip(("dx", "dscale", "dbias"), got, want):
        close(host(a), b, what=name)


@pytest.mark.parametrize("shape", [(32, 64, 112, 112), (64, 8, 56, 56), (3, 2, 300, 300), (40, 5, 64, 64)])
def test_batchnorm_backward_channels_beyond_a_cluster(oracle, shape):
    """Channels too large for a cluster of 8 CTAs go to the streaming kernel
    (ticketed items, totals exchanged through counters in global memory): all
    three mask modes against the oracle, float mask == bit record bit for bit,
    two calls in a row identical, and no fault recorded."""
    import ctypes
    from singa_b200 import _lib
    L = _lib.lib()
    N, C = shape[0], shape[1]
    HW = shape[2] * shape[3]
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    x = torch.randn(shape, device="cuda", generator=g) * 1.5 + 0.3
    dy = torch.randn(shape, device="cuda", generator=g) * 1e-2
    rin = torch.randn(shape, device="cuda", generator=g)
    rin.view(-1)[::7] = 0.0
    scale = torch.rand(C, device="cuda", generator=g) + 0.5
    var, mean = torch.var_mean(x, dim=(0, 2, 3), unbiased=False)
    invstd, mean = torch.rsqrt(var + 1e-5).contiguous(), mean.contiguous()
    n = x.numel()
    s = torch.cuda.current_stream().cuda_stream
    rec = torch.zeros(L.sgb_relu_mask_bytes(n), dtype=torch.uint8, device="cuda")
    y = torch.empty_like(rin)
    _lib.call("sgb_relu_forward_mask_f32", rin.data_ptr(), y.data_ptr(), rec.data_ptr(), n, s)
    ws = torch.empty(max(L.sgb_bn_backward_workspace_bytes(N, C, HW), 256), dtype=torch.uint8, device="cuda")
    outs = {}
    for mode in (0, 1, 2):
        runs = []
        for _ in range(2):
            dx = torch.full(shape, float("nan"), device="cuda")
            ds, db = torch.empty(C, device="cuda"), torch.empty(C, device="cuda")
            tail = [scale.data_ptr(), mean.data_ptr(), invstd.data_ptr(), dx.data_ptr(), ds.data_ptr(), db.data_ptr(),
                    N, C, HW, ws.data_ptr(), ws.numel(), s]
            if mode == 0:
                _lib.call("sgb_bn_backward_f32", x.data_ptr(), dy.data_ptr(), *tail)
            elif mode == 1:
                _lib.call("sgb_bn_relu_backward_f32", x.data_ptr(), dy.data_ptr(), rin.data_ptr(), *tail)
            else:
                _lib.call("sgb_bn_relu_backward_mask_f32", x.data_ptr(), dy.data_ptr(), rec.data_ptr(), *tail)
            torch.cuda.synchronize()
            runs.append((dx, ds, db))
        assert all(torch.equal(a, b) for a, b in zip(*runs)), ("not repeatable", shape, mode)
        gm = dy if mode == 0 else torch.where(rin > 0, dy, torch.zeros_like(dy))
        want = oracle.bn_backward(gm.cpu().numpy(), x.cpu().numpy(), scale.cpu().numpy(), mean.cpu().numpy(),
                                  invstd.cpu().numpy())
        for name, a, b in zip(("dx", "dscale", "dbias"), runs[0], want):
            close(host(a), b, what="%s %s mode %d" % (name, shape, mode))
        outs[mode] = runs[0]
    assert all(torch.equal(a, b) for a, b in zip(outs[1], outs[2])), ("float mask != bit record", shape)
    flags = ctypes.c_uint(1)
    assert L.sgb_bn_backward_faults(ctypes.byref(flags)) == 0 and flags.value == 0


# --------------------------------------------------------------------- pooling
def test_pooling_goldens(sw, golden):
    for key in ("maxpool_cudnn", "maxpool_api", "avgpool_api"):
        g = golden[key]
        x = np.array(g["x"], np.float32).reshape(g["x_shape"])
        h = sw.CudnnPoolingHandle(dev(x), g["kernel"], g["stride"], g["pad"], is_max=key.startswith("max"))
        y = sw.GpuPoolingForward(h, dev(x))
        np.testing.assert_allclose(host(y).ravel(), np.array(g["y"], np.float32).ravel(), rtol=1e-6)
        dy = np.array(g["dy"], np.float32).reshape(tuple(y.shape))
        dx = sw.GpuPoolingBackward(h, dev(dy), dev(x), y)
        np.testing.assert_allclose(host(dx).ravel(), np.array(g["dx"], np.float32).ravel(), rtol=1e-6)


POOL_CASES = [
    ((64, 32, 24, 24), (2, 2), (2, 2), (0, 0)),      # small CNN
    ((64, 32, 8, 8), (2, 2), (2, 2), (0, 0)),
    ((4, 8, 112, 112), (3, 3), (2, 2), (1, 1)),      # ResNet stem geometry
    ((2, 3, 7, 7), (7, 7), (1, 1), (0, 0)),          # ResNet global average
    ((2, 3, 9, 11), (3, 2), (1, 2), (1, 0)),
    ((1, 1, 5, 5), (3, 3), (1, 1), (1, 1)),
    ((3, 2, 6, 6), (2, 2), (3, 3), (0, 0)),          # stride > kernel: gaps get zero
    ((1, 2, 4, 8192), (2, 2), (2, 2), (0, 0)),       # rows too wide to stage: fallback kernel
    ((2, 3, 300, 40), (3, 3), (2, 2), (1, 1)),       # several bands per plane
    ((2, 3, 38, 20), (3, 3), (2, 2), (1, 1)),        # uneven bands
    ((1, 2, 2, 4), (3, 3), (2, 2), (1, 1)),          # smallest stem-geometry plane
    ((2, 2, 9, 12), (3, 3), (2, 2), (1, 1)),         # odd height: general kernel
]


@pytest.mark.parametrize("case", POOL_CASES)
@pytest.mark.parametrize("is_max", [True, False])
def test_pooling_forward_backward(sw, oracle, case, is_max):
    shape, k, s, p = case
    rng = np.random.default_rng(shape[2] * 7 + shape[3])
    x = rng.standard_normal(shape).astype(np.float32)
    x = np.maximum(x, 0)                     # post-ReLU input: many exact ties at 0
    h = sw.CudnnPoolingHandle(dev(x), k, s, p, is_max=is_max)
    y = sw.GpuPoolingForward(h, dev(x))
    dy = rng.standard_normal(tuple(y.shape)).astype(np.float32)
    dx = host(sw.GpuPoolingBackward(h, dev(dy), dev(x), y))
    if is_max:
        assert np.array_equal(host(y), oracle.maxpool_forward(x, k, s, p))
        want = oracle.maxpool_backward(dy, x, k, s, p)
    else:
        close(host(y), oracle.avgpool_forward(x, k, s, p), what="avg fwd")
        want = oracle.avgpool_backward(dy, x.shape, k, s, p)
    assert np.array_equal(dx.view(np.uint32), want.view(np.uint32)), "pool backward not bit-exact"


@pytest.mark.parametrize("case", POOL_CASES + [((32, 64, 112, 112), (3, 3), (2, 2), (1, 1)),
                                               ((2, 4, 56, 56), (3, 3), (2, 2), (1, 1)),
                                               ((1, 2, 10, 20), (3, 3), (2, 2), (1, 1))])
def test_maxpool_argmax_partner_equals_recomputing_backward(sw, case):
    shape, k, s, p = case
    g = torch.Generator(device="cuda").manual_seed(shape[2] * 11 + shape[3])
    x = torch.relu(torch.randn(shape, device="cuda", generator=g))          # exact ties at 0
    x[0, 0, 0, :] = -3.4028234663852886e38                                   # a row no window may credit
    h = sw.CudnnPoolingHandle(x, k, s, p, is_max=True)
    y = sw.GpuPoolingForward(h, x)
    y2, arg = sw.GpuPoolingForwardArgmax(h, x)
    assert torch.equal(y, y2) and arg.dtype == torch.uint8
    dy = torch.randn(tuple(y.shape), device="cuda", generator=g)
    want = sw.GpuPoolingBackward(h, dy, x, y)
    got = sw.GpuPoolingBackwardArgmax(h, dy, arg)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


def test_maxpool_backward_all_equal_window_goes_to_first(sw):
    x = np.zeros((1, 1, 4, 4), np.float32)
    h = sw.CudnnPoolingHandle(dev(x), (2, 2), (2, 2), (0, 0), True)
    y = sw.GpuPoolingForward(h, dev(x))
    dy = np.arange(1, 5, dtype=np.float32).reshape(1, 1, 2, 2)
    dx = host(sw.GpuPoolingBackward(h, dev(dy), dev(x), y))[0, 0]
    want = np.zeros((4, 4), np.float32)
    want[0, 0], want[0, 2], want[2, 0], want[2, 2] = 1, 2, 3, 4
    assert np.array_equal(dx, want)


# ------------------------------------------------------------------------- SGD
def test_sgd_goldens(sw, golden):
    shape = golden["sgd"]["shape"]
    for case in golden["sgd"]["cases"]:
        w = dev(np.full(shape, case["w"], np.float32))
        g0 = np.full(shape, case["g"], np.float32)
        m = torch.zeros_like(w)
        lr = case["lr"]
        w0 = host(w).copy()
        sw.sgd_update_multi([w], [dev(g0)], [m], lr, momentum=case["momentum"],
                            weight_decay=case["weight_decay"])
        if case["name"] == "weight_decay":
            want = w0 - np.float32(lr) * (g0 + np.float32(0.2) * w0)
        else:
            want = w0 - np.float32(lr) * g0
        np.testing.assert_array_almost_equal(host(w), want, decimal=5)
        if case["name"] == "momentum":
            w1 = host(w).copy()
            sw.sgd_update_multi([w], [dev(g0)], [m], lr, momentum=0.9)
            np.testing.assert_array_almost_equal(host(w), w1 - np.float32(lr) * (g0 + g0 * np.float32(0.9)), decimal=5)


@pytest.mark.parametrize("cfg", [dict(momentum=0.9, weight_decay=1e-5), dict(momentum=0.0, weight_decay=0.0),
                                 dict(momentum=0.9, weight_decay=0.0, dampening=0.1),
                                 dict(momentum=0.9, weight_decay=1e-4, nesterov=True),
                                 dict(momentum=0.9, weight_decay=1e-5, grad_scale=0.125)])
def test_sgd_multi_tensor_matches_oracle_bitwise(sw, oracle, cfg):
    rng = np.random.default_rng(9)
    sizes = [1, 3, 64, 1000, 1023, 1025, 4096, 65537, 9408, 2048 * 3 + 1] + [64] * 90 + [300000]
    ps = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    gs = [(rng.standard_normal(n) * 1e-2).astype(np.float32) for n in sizes]
    ms = [(rng.standard_normal(n) * 1e-2).astype(np.float32) for n in sizes]
    dp, dg, dm = [dev(a) for a in ps], [dev(a) for a in gs], [dev(a) for a in ms]
    scale = cfg.get("grad_scale", 1.0)
    for step in range(2):
        sw.sgd_update_multi(dp, dg, dm, 0.1, momentum=cfg["momentum"], dampening=cfg.get("dampening", 0.0),
                            weight_decay=cfg["weight_decay"], nesterov=cfg.get("nesterov", False), grad_scale=scale)
        for p, g, m in zip(ps, gs, ms):
            gg = (g * np.float32(scale)).astype(np.float32) if scale != 1.0 else g.copy()
            oracle.sgd_update(p, gg, m if cfg["momentum"] else None, 0.1, momentum=cfg["momentum"],
                              dampening=cfg.get("dampening", 0.0), weight_decay=cfg["weight_decay"],
                              nesterov=cfg.get("nesterov", False))
    for a, b in zip(dp, ps):
        assert np.array_equal(host(a).view(np.uint32), b.view(np.uint32))
    if cfg["momentum"]:
        for a, b in zip(dm, ms):
            assert np.array_equal(host(a).view(np.uint32), b.view(np.uint32))


# ---------------------------------------------------------------- pack / unpack
def test_pack_unpack_roundtrip_and_half(sw):
    rng = np.random.default_rng(4)
    sizes = [5, 1000, 64, 0, 4096, 3, 2359296 // 8, 77] + [256] * 100
    ts = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    total = sum(sizes)
    flat = torch.zeros(total + 16, device="cuda")
    d = [dev(a) for a in ts]
    sw.pack(d, flat, offset=8)
    want = np.concatenate(ts)
    assert np.array_equal(host(flat)[8:8 + total], want)
    assert host(flat)[:8].sum() == 0 and host(flat)[8 + total:].sum() == 0
    outs = [torch.zeros_like(t) for t in d]
    sw.unpack(flat, outs, offset=8)
    for a, b in zip(outs, ts):
        assert np.array_equal(host(a), b)
    sw.unpack(flat, outs, offset=8, scale=0.25)
    for a, b in zip(outs, ts):
        assert np.array_equal(host(a), b * np.float32(0.25))
    half = torch.zeros(total + 16, device="cuda", dtype=torch.float16)
    sw.pack(d, half, offset=3)
    assert np.array_equal(host(half)[3:3 + total].view(np.uint16), want.astype(np.float16).view(np.uint16))
    sw.unpack(half, outs, offset=3, scale=0.5)
    for a, b in zip(outs, ts):
        assert np.array_equal(host(a), b.astype(np.float16).astype(np.float32) * np.float32(0.5))
