"""GPU parity of the elementwise family against the CPU oracle (bit-exact)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 3, 4, 5, 31, 32, 33, 1023, 1024, 1025, 4099, 65536 + 7, 1 << 20, (1 << 22) + 13]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32 if a.dtype.itemsize == 4 else np.uint16)


@pytest.fixture(scope="module")
def sw():
    from singa_b200 import singa_wrap
    return singa_wrap


def rand_with_zeros(rng, n):
    x = rng.standard_normal(n).astype(np.float32)
    if n:
        x[rng.integers(0, n, max(1, n // 7))] = 0.0
        x[rng.integers(0, n, max(1, n // 11))] = -0.0
    return x


@pytest.mark.parametrize("n", SIZES)
def test_relu_forward_backward_bit_exact(sw, oracle, n):
    rng = np.random.default_rng(n)
    x = rand_with_zeros(rng, n)
    dy = rng.standard_normal(n).astype(np.float32)
    y = host(sw.ReLU(dev(x)))
    dx = host(sw.ReLUBackward(dev(dy), dev(x)))
    assert np.array_equal(bits(y), bits(oracle.relu(x)))
    assert np.array_equal(bits(dx), bits(oracle.relu_backward(dy, x)))


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_relu_backward_misaligned_pointers(sw, oracle, offset):
    rng = np.random.default_rng(offset)
    n = 10007
    x = rand_with_zeros(rng, n + 8)
    dy = rng.standard_normal(n + 8).astype(np.float32)
    dx = sw.ReLUBackward(dev(dy)[offset:offset + n], dev(x)[offset:offset + n])
    want = oracle.relu_backward(dy[offset:offset + n], x[offset:offset + n])
    assert np.array_equal(bits(host(dx)), bits(want))


def test_relu_golden(sw, golden):
    g = golden["relu"]
    x = np.array(g["x"], np.float32).reshape(g["shape"])
    dy = np.ones(g["shape"], np.float32)
    assert np.array_equal(host(sw.ReLU(dev(x))), np.maximum(x, 0))
    assert np.array_equal(host(sw.ReLUBackward(dev(dy), dev(x))), (x > 0) * dy)


@pytest.mark.parametrize("n", [1, 7, 8, 9, 1000, 100003])
def test_relu_half_rules(sw, oracle, n):
    rng = np.random.default_rng(n)
    x = rand_with_zeros(rng, n).astype(np.float16)
    dy = rng.standard_normal(n).astype(np.float16)
    y = host(sw.ReLU(dev(x)))
    dx = host(sw.ReLUBackward(dev(dy), dev(x)))
    assert np.array_equal(bits(y), bits(np.where(x > 0, x, np.float16(0))))
    assert np.array_equal(bits(dx), bits(oracle.relu_backward_f16(dy, x)))


@pytest.mark.parametrize("n", [5, 4096, 1 << 20])
def test_join_and_fused_join_relu(sw, oracle, n):
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    x = rand_with_zeros(rng, n)
    ta = dev(a)
    sw.iAdd(ta, dev(b))
    assert np.array_equal(bits(host(ta)), bits(a + b))
    fused = host(sw.AddReLUBackward(dev(a), dev(b), dev(x)))
    assert np.array_equal(bits(fused), bits(oracle.relu_backward(a + b, x)))


def test_binary_scalar_unary_family(sw):
    rng = np.random.default_rng(5)
    n = 50021
    a = rng.standard_normal(n).astype(np.float32)
    b = (rng.standard_normal(n).astype(np.float32) + 3.0)
    ops = {"add": a + b, "sub": a - b, "mul": a * b, "div": a / b,
           "gt": (a > b), "ge": (a >= b), "eq": (a == b), "lt": (a < b), "le": (a <= b)}
    for op, want in ops.items():
        got = host(sw.binary(op, dev(a), dev(b)))
        assert np.array_equal(bits(got), bits(want.astype(np.float32))), op
    s = np.float32(0.37)
    sops = {"add": a + s, "mul": a * s, "rdiv": s / b, "gt": a > s, "le": a <= s, "threshold": a < s}
    for op, want in sops.items():
        src = b if op == "rdiv" else a
        got = host(sw.scalar(op, dev(src), float(s)))
        assert np.array_equal(bits(got), bits(want.astype(np.float32))), op
    # transcendental members: same libdevice functions as the reference, checked to 2 ulp-ish
    for op, fn in {"exp": np.exp, "tanh": np.tanh, "sqrt": lambda v: np.sqrt(np.abs(v)),
                   "sigmoid": lambda v: 1 / (1 + np.exp(-v)), "square": np.square,
                   "abs": np.abs, "sign": np.sign}.items():
        src = np.abs(a) if op == "sqrt" else a
        got = host(sw.unary(op, dev(src)))
        np.testing.assert_allclose(got, fn(src.astype(np.float64)), rtol=2e-6, atol=1e-7, err_msg=op)
    got = host(sw.Clamp(dev(a), -0.5, 0.25))
    assert np.array_equal(got, np.clip(a, -0.5, 0.25))


@pytest.mark.parametrize("n", [1, 7, 8, 9, 4095, 1 << 20, (1 << 20) + 5])
def test_casts(sw, n):
    rng = np.random.default_rng(n)
    a = (rng.standard_normal(n) * 100).astype(np.float32)
    h = host(sw.AsType(dev(a), torch.float16))
    assert np.array_equal(bits(h), bits(a.astype(np.float16)))       # round-to-nearest-even
    f = host(sw.AsType(dev(h), torch.float32))
    assert np.array_equal(bits(f), bits(h.astype(np.float32)))
    i = host(sw.AsType(dev(a), torch.int32))
    assert np.array_equal(i, a.astype(np.int32))                      # truncation
    assert np.array_equal(host(sw.AsType(dev(i), torch.float32)), i.astype(np.float32))


def test_set_axpy_transform(sw):
    t = torch.empty(1000003, device="cuda")
    sw.SetValue(t, 1.5)
    assert bool((t == 1.5).all())
    rng = np.random.default_rng(2)
    x = rng.standard_normal(70001).astype(np.float32)
    y = rng.standard_normal(70001).astype(np.float32)
    ty = dev(y)
    sw.Axpy(-0.05, dev(x), ty)
    want = (np.float64(np.float32(-0.05)) * x.astype(np.float64) + y).astype(np.float32)  # one rounding (fma)
    assert np.array_equal(bits(host(ty)), bits(want))
    ty = dev(y)
    sw.Axpy(dev(np.array([0.9], np.float32)), dev(x), ty)
    want = (np.float64(np.float32(0.9)) * x.astype(np.float64) + y).astype(np.float32)
    assert np.array_equal(bits(host(ty)), bits(want))
    # broadcast of a (1,) tensor to a parameter shape, and a transposed view
    one = dev(np.array([0.9], np.float32))
    assert bool((sw.Transform(one, [3, 5], [0, 0]) == 0.9).all())
    m = rng.standard_normal((4, 6)).astype(np.float32)
    tr = host(sw.Transform(dev(m), [6, 4], [1, 6]))
    assert np.array_equal(tr, m.T)


def test_tensor_math_fixture_goldens(sw, golden):
    """The CUDA variants of the reference's tensor-math tests on its own fixture
    (test_tensor_math.cc) and the legacy Dense bias gradient (test_dense.cc)."""
    g = golden["tensor_math"]
    a = np.array(g["dat1"], np.float32)
    m = a.reshape(g["shape"])
    shifted = sw.scalar("add", dev(a), -g["relu_shift"])
    np.testing.assert_array_equal(host(sw.ReLU(shifted))[:3], np.array(g["relu_expect_first3"], np.float32))
    np.testing.assert_array_equal(host(sw.SumRows(dev(m))), m.sum(axis=0))
    np.testing.assert_array_equal(host(sw.SumColumns(dev(m))), m.sum(axis=1))
    # L2 = Nrm2 / size
    np.testing.assert_allclose(host(sw.Nrm2(dev(a)))[0] / a.size, np.sqrt((a * a).sum()) / a.size, rtol=1e-6)
    # MultColumn (diag(v) * M), MultRow and DivRow (M * diag(v), M * diag(1/v))
    vc = np.array(g["mult_column_x"], np.float32)
    np.testing.assert_array_equal(host(sw.DGMM(False, dev(m), dev(vc))), m * vc[:, None])
    vr = np.array(g["mult_row_x"], np.float32)
    np.testing.assert_array_equal(host(sw.DGMM(True, dev(m), dev(vr))), m * vr[None, :])
    inv = sw.scalar("rdiv", dev(np.array(g["div_row_x"], np.float32)), 1.0)      # 1 / v, as DivRow forms it
    np.testing.assert_allclose(host(sw.DGMM(True, dev(m), inv)), m / vr[None, :], rtol=1e-6)
    rm = np.array(g["row_max_in"], np.float32).reshape(2, 2)
    np.testing.assert_array_equal(host(sw.RowMax(dev(rm))), np.array(g["row_max_expect"], np.float32))
    si = np.array(g["soft_in"], np.float32)
    np.testing.assert_allclose(host(sw.unary("softplus", dev(si))), [np.log(2.0), np.log(np.e + 1.0)], atol=1e-5)
    np.testing.assert_array_equal(host(sw.unary("softsign", dev(si))), np.array(g["softsign_expect"], np.float32))
    # strided Exp: exp of the fixture seen as (1,3,2), written through a (1,2,0)-transposed (2,1,3) tensor
    # = the contiguous materialisation of the transposed view; the test checks three entries
    y = host(sw.unary("exp", sw.Transform(dev(a), (2, 1, 3), (1, 2, 2))))
    ref = np.exp(a.reshape(1, 3, 2)).transpose(2, 0, 1).reshape(-1)
    np.testing.assert_allclose(y.reshape(-1), ref, rtol=1e-6)
    for out_i, dat_i in g["exp_stride_checks"]:
        np.testing.assert_allclose(y.reshape(-1)[out_i], np.exp(a[dat_i]), rtol=1e-5)
    d = golden["dense_bias_grad"]
    dy = np.array(d["dy"], np.float32).reshape(d["shape"])
    np.testing.assert_array_equal(host(sw.SumRows(dev(dy))), dy.sum(axis=0))


def test_astype_goldens(sw, golden):
    g = golden["astype"]
    t = sw.AsType(dev(np.array(g["float_in"], np.float32)), torch.int32)
    np.testing.assert_array_equal(host(t), np.array(g["int_expect"], np.int32))
    t = sw.AsType(dev(np.array(g["int_in"], np.int32)), torch.float32)
    np.testing.assert_array_equal(host(t), np.array(g["float_expect"], np.float32))
    rng = np.random.default_rng(3)
    f = (rng.random((2, 3)) * 10 - 5).astype(np.float32)           # the python test's distribution
    i = sw.AsType(dev(f), torch.int32)
    np.testing.assert_array_equal(host(i), f.astype(np.int32))
    np.testing.assert_array_equal(host(sw.AsType(i, torch.float32)), f.astype(np.int32).astype(np.float32))


def test_softmax_cudnn_layer_golden(sw, golden):
    g = golden["softmax_cudnn"]
    for shape in g["shapes"]:
        x = np.array(g["x"], np.float32).reshape(shape)
        e = np.exp(x.astype(np.float64))
        np.testing.assert_allclose(host(sw.SoftMax(dev(x))), e / e.sum(axis=1, keepdims=True), rtol=1e-6)


def test_softmax_axis_goldens(sw, golden):
    rng = np.random.default_rng(0)
    for shape, axis, two_d in golden["softmax_axis"]["cases"]:
        x = (rng.random(shape) + 1000).astype(np.float32)
        x2 = x.reshape(two_d)
        e = np.exp(x2 - x2.max())
        want = (e / e.sum(axis=1, keepdims=True)).reshape(shape)
        np.testing.assert_array_almost_equal(host(sw.SoftMax(dev(x), axis)), want)


def test_cpu_tensor_is_rejected(sw):
    with pytest.raises(ValueError):
        sw.ReLU(torch.zeros(4))
