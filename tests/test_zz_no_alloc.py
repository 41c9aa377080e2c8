"""The allocation-free batch-norm backward entry point (built-in scratch).

Meant for callers that cannot obtain device memory at call time - for example
an operator that runs while a framework's own memory pool owns the whole GPU,
or a thread that must not cause the device-wide synchronisation an allocation
can imply - and therefore have no workspace to pass.  The test calls it
through the C ABI and compares it with the regular entry point (which is given
a workspace) AND with the CPU oracle, on two calls in a row with different
inputs, so that scratch contents left behind by the first call would show up
in the second.

This file sorts last on purpose: a run that stops at the first failure has
already gone through every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 1e-5        # the tolerance used for fp32 reductions elsewhere in the suite


def rel(a, b):
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def both_paths(lib, shape, seed):
    from singa_b200 import _lib
    N, C = shape[0], shape[1]
    HW = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, device="cuda", generator=g) * 1.5 + 0.2
    dy = torch.randn(shape, device="cuda", generator=g) * 1e-2
    scale = torch.rand(C, device="cuda", generator=g) + 0.5
    flat = x.reshape(N, C, HW)
    var, mean = torch.var_mean(flat, dim=(0, 2), unbiased=False)
    invstd = torch.rsqrt(var).contiguous()
    mean = mean.contiguous()
    s = torch.cuda.current_stream().cuda_stream
    outs = []
    for name in ("sgb_bn_backward_f32", "sgb_bn_backward_noalloc_f32"):
        dx, ds, db = torch.empty_like(x), torch.empty(C, device="cuda"), torch.empty(C, device="cuda")
        args = [x.data_ptr(), dy.data_ptr(), scale.data_ptr(), mean.data_ptr(), invstd.data_ptr(),
                dx.data_ptr(), ds.data_ptr(), db.data_ptr(), N, C, HW]
        if name == "sgb_bn_backward_f32":
            ws = torch.empty(max(lib.sgb_bn_backward_workspace_bytes(N, C, HW), 256), dtype=torch.uint8,
                             device="cuda")
            args += [ws.data_ptr(), ws.numel()]
        _lib.call(name, *args, s)
        outs.append((dx, ds, db))
    torch.cuda.synchronize()
    from oracle import cpu
    x4 = x.reshape(N, C, HW, 1).cpu().numpy()
    want = cpu.bn_backward(dy.reshape(N, C, HW, 1).cpu().numpy(), x4, scale.cpu().numpy(), mean.cpu().numpy(),
                           invstd.cpu().numpy())
    outs.append(tuple(torch.from_numpy(np.ascontiguousarray(w)).reshape(o.shape).cuda()
                      for w, o in zip(want, outs[0])))
    return outs


@pytest.mark.parametrize("shape", [(32, 64, 56, 56), (8, 5, 7, 7), (32, 64, 112, 112), (16, 100)])
def test_noalloc_matches_regular_entry_point_twice_in_a_row(shape):
    from singa_b200 import _lib
    lib = _lib.lib()
    for call in range(2):                      # second call: new inputs, same built-in scratch
        regular, noalloc, oracle = both_paths(lib, shape, seed=17 * (call + 1) + shape[1])
        for name, a, b, c in zip(("dx", "dscale", "dbias"), noalloc, regular, oracle):
            assert rel(a, b) <= RTOL, (shape, call, name, rel(a, b))
            assert rel(a, c) <= 2 * RTOL, ("vs oracle", shape, call, name, rel(a, c))


def test_noalloc_rejects_more_channels_than_the_scratch_holds():
    from singa_b200 import _lib
    lib = _lib.lib()
    C = 4097
    x = torch.zeros(2, C, 1, 1, device="cuda")
    v = torch.ones(C, device="cuda")
    dx, ds, db = torch.full_like(x, 7.0), torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    status = lib.sgb_bn_backward_noalloc_f32(x.data_ptr(), x.data_ptr(), v.data_ptr(), v.data_ptr(), v.data_ptr(),
                                             dx.data_ptr(), ds.data_ptr(), db.data_ptr(), 2, C, 1,
                                             torch.cuda.current_stream().cuda_stream)
    assert status == -9                                   # SGB_ERR_LIMIT
    assert b"built-in scratch" in lib.sgb_status_string(status)
    torch.cuda.synchronize()
    assert bool((dx == 7.0).all())                        # nothing was launched
    # the limit itself is accepted, and its values are right
    regular, noalloc, oracle = both_paths(lib, (4, 4096, 3, 3), seed=5)
    for name, a, b, c in zip(("dx", "dscale", "dbias"), noalloc, regular, oracle):
        assert rel(a, b) <= RTOL, ("C = 4096", name, rel(a, b))
        assert rel(a, c) <= 2 * RTOL, ("C = 4096 vs oracle", name, rel(a, c))
