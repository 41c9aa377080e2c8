"""Oracle statement of the capacity-bounded threshold exchange (the GPU path is
checked against it in tests/dist_worker.py): with ample capacity it is the
reference's exchange; with a tight one nothing is lost while a residual is
kept - what is not sent stays behind and goes out later."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def oc():
    from oracle import build, comm
    build.build_oracle()
    return comm


def grads(world, n, seed):
    return [(np.random.default_rng(seed + 31 * r).standard_normal(n) * 1e-3).astype(np.float32) for r in range(world)]


@pytest.mark.parametrize("world", [1, 2, 3])
def test_ample_capacity_is_the_unbounded_exchange(oc, world):
    n, thr = 20011, 2e-3
    a1 = [np.zeros(n, np.float32) for _ in range(world)]
    a2 = [np.zeros(n, np.float32) for _ in range(world)]
    for step in range(3):
        gs = grads(world, n, 100 * step)
        d1, a1, _ = oc.sparse_threshold_step(gs, a1, thr)
        d2, a2, held = oc.sparse_threshold_bounded_step(gs, a2, thr, n)
        assert held == [0] * world
        assert np.array_equal(d1.view(np.uint32), d2.view(np.uint32))
        for x, y in zip(a1, a2):
            assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


def test_tight_capacity_sends_the_first_entries_and_keeps_the_rest(oc):
    n, thr, cap, world = 20011, 2e-3, 40, 2
    accs = [np.zeros(n, np.float32) for _ in range(world)]
    gs = grads(world, n, 7)
    dense, accs2, held = oc.sparse_threshold_bounded_step(gs, accs, thr, cap)
    for r in range(world):
        sel = np.flatnonzero(np.abs(gs[r]) >= np.float32(thr))
        assert held[r] == len(sel) - cap > 0
        assert np.array_equal(np.flatnonzero(accs2[r] == 0), np.sort(sel[:cap]))       # exactly the sent ones left
        assert np.array_equal(accs2[r][sel[cap:]], gs[r][sel[cap:]])                 # held back, bit for bit
    want = np.zeros(n, np.float32)
    for r in range(world):
        sel = np.flatnonzero(np.abs(gs[r]) >= np.float32(thr))[:cap]
        want[sel] += gs[r][sel]
    assert np.array_equal(dense.view(np.uint32), want.view(np.uint32))
    # a later step with zero gradients drains what was held back, lowest indices first
    zeros = [np.zeros(n, np.float32) for _ in range(world)]
    dense2, accs3, held2 = oc.sparse_threshold_bounded_step(zeros, accs2, thr, cap)
    assert all(h2 == max(h - cap, 0) for h, h2 in zip(held, held2))
    assert int((dense2 != 0).sum()) > 0


def test_without_a_residual_the_excess_is_dropped(oc):
    n, thr, cap = 5003, 2e-3, 10
    gs = grads(1, n, 3)
    dense, accs, held = oc.sparse_threshold_bounded_step(gs, None, thr, cap)
    assert accs is None and held[0] > 0
    assert int((dense != 0).sum()) == cap
