"""GPU parity of the sparsification kernels against the CPU oracle: payloads
(1-based index, value) and residuals are compared bit for bit; top-K index sets
with ties broken by lower index, in both key modes."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 5, 4095, 4096, 4097, 100003, (1 << 20) + 3, 5000000]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def sw():
    from singa_b200 import singa_wrap
    return singa_wrap


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("corr", [True, False])
def test_threshold_payload_and_residual(sw, oracle, n, corr):
    rng = np.random.default_rng(n)
    g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    acc = (rng.standard_normal(n) * 1e-3).astype(np.float32) if corr else None
    if n > 10:
        g[3] = 0.0
        if corr:
            acc[3] = 0.0            # exact zero: never sent, even with thr == 0
    for thr in (2e-3, 0.0):
        d_acc = dev(acc) if corr else None
        idx, val = sw.sparse_threshold(dev(g), d_acc, thr)
        w_idx, w_val, w_acc = oracle.sparse_threshold(g, acc, thr)
        assert np.array_equal(idx.cpu().numpy(), w_idx)
        assert np.array_equal(val.cpu().numpy().view(np.uint32), w_val.view(np.uint32))
        if corr:
            assert np.array_equal(d_acc.cpu().numpy().view(np.uint32), w_acc.view(np.uint32))


def test_threshold_nothing_and_everything(sw):
    g = dev(np.full(10000, 0.5, np.float32))
    idx, val = sw.sparse_threshold(g, None, 1.0)
    assert idx.numel() == 0
    idx, val = sw.sparse_threshold(g, None, 0.05)
    assert np.array_equal(idx.cpu().numpy(), np.arange(1, 10001, dtype=np.int32))


def test_threshold_selector_repeats_on_a_multi_wave_size(sw):
    """Many calls in a row on a size of several waves of tiles give the same
    payload every time, unaligned buffers included."""
    n = 10000019
    rng = np.random.default_rng(1)
    g_host = (rng.standard_normal(n + 1) * 1e-3).astype(np.float32)
    for shift in (0, 1):                       # shift 1: 4-byte aligned only (scalar loads)
        g = dev(g_host)[shift:shift + n]
        first = None
        for _ in range(5):
            idx, val = sw.sparse_threshold(g, None, 2e-3)
            got = (idx.cpu().numpy(), val.cpu().numpy().view(np.uint32))
            if first is None:
                first = got
                want = np.flatnonzero(np.abs(g_host[shift:shift + n]) >= np.float32(2e-3)) + 1
                assert np.array_equal(got[0], want.astype(np.int32))
            assert np.array_equal(got[0], first[0]) and np.array_equal(got[1], first[1])


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("mode", ["magnitude", "compat"])
def test_topk_index_set_values_residual(sw, n, mode):
    from oracle import comm
    rng = np.random.default_rng(n + 17)
    scale = 1e-3 if mode == "magnitude" else 3.0     # compat keys are |trunc(s)|
    g = (rng.standard_normal(n) * scale).astype(np.float32)
    acc = (rng.standard_normal(n) * scale).astype(np.float32)
    if n > 100:                                        # plant exact ties around the cut
        g[10:60] = np.float32(0.25 * scale)
        acc[10:60] = 0.0
    for ratio in (0.01, 0.3, 1.0):
        k = comm.topk_count(ratio, n)
        assert k == sw.topk_count(ratio, n)
        d_acc = dev(acc)
        idx, val = sw.sparse_topk(dev(g), d_acc, k, mode)
        s = (g + acc).astype(np.float32)
        sel = comm.topk_select(s, k, mode)
        assert np.array_equal(idx.cpu().numpy().astype(np.int64) - 1, sel), (n, mode, ratio)
        assert np.array_equal(val.cpu().numpy().view(np.uint32), s[sel].view(np.uint32))
        want_acc = s.copy()
        want_acc[sel] = 0.0
        assert np.array_equal(d_acc.cpu().numpy().view(np.uint32), want_acc.view(np.uint32))


def test_topk_all_keys_tie_takes_lowest_indices(sw):
    # N(0, 1e-3) gradients under the reference comparator: every key is 0.
    rng = np.random.default_rng(0)
    n = 1000003
    g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    k = sw.topk_count(0.01, n)
    idx, val = sw.sparse_topk(dev(g), None, k, "compat")
    assert np.array_equal(idx.cpu().numpy(), np.arange(1, k + 1, dtype=np.int32))
    assert np.array_equal(val.cpu().numpy(), g[:k])


def test_topk_count_is_fp32_arithmetic(sw):
    assert sw.topk_count(0.01, 100000000) == 1000000
    assert sw.topk_count(1.0, 100) == 100
    assert sw.topk_count(0.05, 25557032) == int(np.ceil(np.float32(0.05) * np.float32(25557032)))


def test_scatter_add_ranks_in_order(sw, oracle):
    rng = np.random.default_rng(5)
    n = 200000
    dst = np.zeros(n, np.float32)
    d = dev(dst)
    for r in range(4):
        idx = np.sort(rng.choice(n, 5000, replace=False)).astype(np.int32) + 1
        idx[::97] = 0                                   # padding entries are skipped
        val = rng.standard_normal(5000).astype(np.float32)
        sw.scatter_add(d, dev(idx), dev(val))
        oracle.scatter_add(dst, idx, val)
    assert np.array_equal(d.cpu().numpy().view(np.uint32), dst.view(np.uint32))
