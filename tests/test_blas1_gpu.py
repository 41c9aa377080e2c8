"""BLAS-1 style reductions, DGMM, fp16 axpy / softmax and the strided gather in
fp16 against numpy (1e-5 relative for fp32 sums, exact for index results)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sw():
    from singa_b200 import singa_wrap
    return singa_wrap


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n", [1, 3, 4, 5, 1023, 4099, 1 << 20, (1 << 22) + 3])
@pytest.mark.parametrize("offset", [0, 1])
def test_dot_asum_nrm2(sw, n, offset):
    rng = np.random.default_rng(n + offset)
    x = rng.standard_normal(n + offset).astype(np.float32)
    y = rng.standard_normal(n + offset).astype(np.float32)
    dx, dy = dev(x)[offset:], dev(y)[offset:]          # offset 1: not 16-byte aligned
    x, y = x[offset:].astype(np.float64), y[offset:].astype(np.float64)
    tol = 1e-5
    got = sw.Dot(dx, dy).item()
    assert abs(got - (x * y).sum()) <= tol * np.abs(x * y).sum()
    assert abs(sw.Asum(dx).item() - np.abs(x).sum()) <= tol * np.abs(x).sum()
    assert abs(sw.Nrm2(dx).item() - np.sqrt((x * x).sum())) <= tol * np.sqrt((x * x).sum())
    # run-to-run identical
    assert sw.Dot(dx, dy).item() == got


@pytest.mark.parametrize("n", [1, 2, 33, 1025, 100003, (1 << 21) + 1])
def test_amax_amin_first_occurrence(sw, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    if n > 40:
        x[7], x[n - 3] = -9.0, 9.0                     # equal magnitudes: the first wins
        x[11], x[n // 2] = 0.0, -0.0
    a = np.abs(x)
    assert sw.Amax(dev(x)).item() == int(np.argmax(a))
    assert sw.Amin(dev(x)).item() == int(np.argmin(a))


@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (257, 130), (1000, 33)])
def test_dgmm(sw, shape):
    rng = np.random.default_rng(sum(shape))
    M = rng.standard_normal(shape).astype(np.float32)
    vr, vc = rng.standard_normal(shape[0]).astype(np.float32), rng.standard_normal(shape[1]).astype(np.float32)
    assert np.array_equal(sw.DGMM(True, dev(M), dev(vc)).cpu().numpy(), M * vc[None, :])
    assert np.array_equal(sw.DGMM(False, dev(M), dev(vr)).cpu().numpy(), M * vr[:, None])


@pytest.mark.parametrize("n", [1, 7, 4099, 1 << 20])
def test_axpy_half(sw, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float16)
    y = rng.standard_normal(n).astype(np.float16)
    alpha = np.float32(-0.37)
    # one fp32 fused multiply-add (exact product and sum, rounded to fp32), then one rounding to fp16
    want = (np.float64(alpha) * x.astype(np.float64) + y.astype(np.float64)).astype(np.float32).astype(np.float16)
    for a in (float(alpha), dev(np.array([alpha], np.float32))):
        out = dev(y).clone()
        sw.Axpy(a, dev(x), out)
        assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_softmax_half_and_transform_half(sw):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((33, 1000)) * 3).astype(np.float16)
    y = sw.SoftMax(dev(x)).cpu().numpy().astype(np.float64)
    e = np.exp(x.astype(np.float64) - x.astype(np.float64).max(1, keepdims=True))
    want = e / e.sum(1, keepdims=True)
    assert np.abs(y - want).max() <= 1e-3 * want.max()
    src = rng.standard_normal((5, 1, 7)).astype(np.float16)
    got = sw.Transform(dev(src.reshape(-1)), (7, 3, 5), (1, 0, 7)).cpu().numpy()
    want = np.broadcast_to(src, (5, 3, 7)).transpose(2, 1, 0)
    assert np.array_equal(got.view(np.uint16), np.ascontiguousarray(want).view(np.uint16))
