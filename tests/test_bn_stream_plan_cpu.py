"""Host arithmetic of the streaming batch-norm backward kernel: how an
(N, C, HW) problem is cut into pieces, items and staging slots.  Pure host
logic behind the C ABI (no device work), so it runs without a GPU."""
import ctypes
import itertools

import pytest


@pytest.fixture(scope="module")
def lib():
    from singa_b200 import _lib
    return _lib.lib()


def plan(lib, N, C, HW, mask):
    out = (ctypes.c_int * 6)()
    ok = lib.sgb_bn_backward_stream_plan(N, C, HW, mask, out)
    assert ok in (0, 1)
    return dict(zip(("P", "Lp", "S", "parts", "ctas_per_sm", "arrays"), out)) if ok else None


SHAPES = [(32, 64, 112 * 112), (32, 256, 56 * 56), (32, 512, 28 * 28), (32, 1024, 14 * 14), (64, 8, 56 * 56),
          (3, 2, 300 * 300), (40, 5, 64 * 64), (1, 1, 4), (2, 4096, 4), (7, 130, 36), (128, 3, 224 * 224),
          (5, 3, 400), (32, 64, 28 * 28), (256, 16, 8 * 8)]


@pytest.mark.parametrize("shape", SHAPES)
def test_partition_covers_the_channel_and_fits_the_machine(lib, shape):
    N, C, HW = shape
    plans = [plan(lib, N, C, HW, m) for m in (0, 1, 2)]
    if plans[0] is None:
        assert plans == [None, None, None]
        return
    for mask, p in enumerate(plans):
        assert p is not None, (shape, mask)
        assert p["P"] * p["Lp"] == HW                      # pieces tile a plane exactly
        assert p["Lp"] % 4 == 0 and p["Lp"] * 4 <= 25088   # 16-byte runs, a piece fits a slot
        pieces = N * p["P"]
        assert 1 <= p["S"] <= pieces
        assert p["parts"] == -(-pieces // p["S"]) <= 64    # items per channel; bounds the workspace
        assert p["arrays"] == (3 if mask == 1 else 2)
        slot = p["arrays"] * p["S"] * p["Lp"] * 4
        assert 2 <= p["ctas_per_sm"] <= 16
        assert p["ctas_per_sm"] * slot <= 228 * 1024       # the slots of an SM fit its shared memory
        assert lib.sgb_bn_backward_workspace_bytes(N, C, HW) >= C * p["parts"] * 8
    # the cut (and with it the order of the additions) does not depend on the mask mode
    for key in ("P", "Lp", "S", "parts"):
        assert len({p[key] for p in plans}) == 1, (shape, key)


@pytest.mark.parametrize("shape", [(32, 2048, 49), (4, 8, 6), (32, 5000, 64), (0, 4, 16), (4, 0, 16), (4, 4, 0)])
def test_shapes_the_streaming_form_does_not_take(lib, shape):
    for mask in (0, 1, 2):
        assert plan(lib, *shape, mask) is None


def test_many_shapes_keep_the_invariants(lib):
    for N, C, hw in itertools.product((1, 2, 31, 32, 64, 200), (1, 3, 64, 1000, 4096), (4, 64, 196, 784, 3136, 12544, 50176)):
        p = plan(lib, N, C, hw, 0)
        if p is None:
            continue
        assert p["P"] * p["Lp"] == hw and p["Lp"] % 4 == 0
        assert p["parts"] == -(-(N * p["P"]) // p["S"]) <= 64
