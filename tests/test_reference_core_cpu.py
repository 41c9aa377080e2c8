"""The CPU restatement (oracle/oracle.c) against the code it restates: the
reference's own lang::Cpp tensor back end, compiled unmodified from its source
tree into oracle/_ref/libref_core.so (oracle/ref_core_build.py).  Also the
whole backward + update step of the MLP configuration through the reference's
Tensor functions against the oracle executor."""
import numpy as np
import pytest

from oracle import ref_core, ref_core_build


def _have_core():
    try:
        return ref_core_build.build_ref_core() is not None
    except Exception:
        return False


pytestmark = pytest.mark.skipif(not _have_core(), reason="reference tree absent and libref_core.so not built")


def test_elementwise_and_loss_functions_match_the_reference_cpu_code(oracle):
    rng = np.random.default_rng(3)
    dy = rng.standard_normal(10007).astype(np.float32)
    x = rng.standard_normal(10007).astype(np.float32)
    x[::7] = 0.0                                            # the boundary of the > 0 rule
    assert np.array_equal(ref_core.relu_backward(dy, x), oracle.relu_backward(dy, x))
    for rows, cols in ((256, 10), (64, 10), (32, 1000)):
        logits = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
        p_ref, p = ref_core.softmax(logits), oracle.softmax(logits)
        np.testing.assert_allclose(p, p_ref, rtol=1e-5, atol=1e-12)   # a row sum: 1e-5 relative
        t = rng.integers(0, cols, rows).astype(np.int32)
        assert np.array_equal(ref_core.cross_entropy(p_ref, t), oracle.cross_entropy_fwd(p_ref, t))
        assert np.array_equal(ref_core.softmax_cross_entropy_bwd(p_ref, t), oracle.softmax_cross_entropy_bwd(p_ref, t))
    m = rng.standard_normal((256, 4096)).astype(np.float32)
    want = m.astype(np.float64).sum(0)
    scale = np.abs(want).max()
    assert np.abs(ref_core.sum_axis0(m) - want).max() <= 1e-5 * scale
    assert np.abs(oracle.sum_rows(m) - want).max() <= 1e-5 * scale
    v = rng.standard_normal(256).astype(np.float32)
    assert abs(ref_core.sum_all(v) - float(oracle.sum_all(v))) <= 1e-5 * np.abs(v).sum()


@pytest.mark.parametrize("momentum,weight_decay", [(0.0, 0.0), (0.9, 0.0), (0.9, 1e-5)])
def test_sgd_chain_matches_the_reference_axpy_sequence(oracle, momentum, weight_decay):
    rng = np.random.default_rng(4)
    n = 5000
    p0 = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32) * np.float32(1e-2)
    m0 = rng.standard_normal(n).astype(np.float32) * np.float32(1e-2)
    p_ref, m_ref = p0.copy(), m0.copy()
    ref_core.sgd(p_ref, g, m_ref, 0.05, momentum, weight_decay)
    p, m = p0.copy(), m0.copy()
    oracle.sgd_update(p, g.copy(), m, 0.05, momentum=momentum, weight_decay=weight_decay)
    np.testing.assert_allclose(p, p_ref, rtol=1e-6, atol=1e-7)
    if momentum:
        np.testing.assert_allclose(m, m_ref, rtol=1e-6, atol=1e-7)


def test_mlp_backward_update_step_matches_the_oracle_executor():
    """Configuration 1's shape family at a reduced size: the reference's Tensor
    functions walk softmax-CE, the bias-gradient reductions, ReLU backward and
    the SGD-momentum chain; the oracle executor walks the same plan."""
    from oracle.path import OraclePath, make_tensors
    from singa_b200.resnet50_path import build_mlp_plan
    dims = (48, 96, 64, 10)
    plan = build_mlp_plan(batch=32, dims=dims)
    t = make_tensors(plan, seed=7)
    L = len(dims) - 1
    mlp = ref_core.MLP(32, dims, lr=0.05, momentum=0.9)
    for i in range(L):
        mlp.set(i, 0, t["fc%d.W" % i])
        mlp.set(i, 1, t["fc%d.b" % i])
    relu_x = [t["relu%d.x" % i] for i in range(L - 1)]
    dgrad = [None] + [t["fc%d.dgrad" % i] for i in range(1, L)]
    wgrad = [t["d:fc%d.W" % i].copy() for i in range(L)]
    ref = OraclePath(plan, t, lr=0.05, momentum=0.9, weight_decay=0.0)
    for _ in range(2):                                      # two steps: the moments matter in the second
        loss = ref_core.mlp_hot_path_step(mlp, t["logits"], t["labels"], relu_x, dgrad, wgrad)
        ref.run_step()
        assert abs(loss - float(t["loss"][0]) / 32) <= 1e-5 * abs(loss)     # the plan keeps the sum, the reference the mean
    for i in range(L):
        for which, name in ((0, "fc%d.W" % i), (1, "fc%d.b" % i), (2, "m:fc%d.W" % i), (3, "m:fc%d.b" % i)):
            got, want = mlp.get(i, which), t[name]
            scale = max(np.abs(want).max(), 1e-30)
            assert np.abs(got - want).max() <= 2e-6 * scale, name
    mlp.close()
