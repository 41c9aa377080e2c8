"""End-to-end parity of the ResNet backward + sync + update step: the GPU
executor against the oracle executor on the same seeded tensors, unfused and
fused plans, eager and CUDA-graph replay."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def close(got, want, rtol, what):
    want = np.asarray(want, np.float64)
    scale = max(np.abs(want).max(), 1e-30)
    err = np.abs(np.asarray(got, np.float64) - want).max()
    assert err <= rtol * scale, "%s: rel err %.3e" % (what, err / scale)


@pytest.mark.parametrize("fused", [False, True, "join_bn"])
@pytest.mark.parametrize("graph", [False, True])
def test_small_resnet_step_matches_oracle(fused, graph):
    from oracle.path import OraclePath
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import build_plan
    plan = build_plan(batch=4, image=64, num_classes=10, fused=bool(fused), blocks=(2, 1, 1, 1),
                      join_bn=fused == "join_bn")
    gpu = HotPathGPU(plan, communicator=None, world=1, seed=5)
    host = gpu.host_copy()
    ref = OraclePath(plan, host)
    steps = 2
    for _ in range(steps):
        ref.run_step()
    if graph:
        gpu.run_step()                      # warm-up = step 1
        g = gpu.capture()                   # capturing does not execute
        g.replay()                          # step 2
    else:
        for _ in range(steps):
            gpu.run_step()
    torch.cuda.synchronize()
    got = gpu.host_copy()
    for name, spec in plan["tensors"].items():
        if spec.kind in ("grad", "pgrad"):
            close(got[name], host[name], 2e-5, name)
    for p in plan["params"]:
        close(got[p], host[p], 1e-6, "param " + p)
        close(got["m:" + p], host["m:" + p], 2e-5, "moment " + p)
    close(got["loss"], host["loss"], 1e-5, "loss")


def test_pool_argmax_record_gives_the_same_step_bitwise():
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import build_plan
    outs = []
    for flag in (False, True):
        plan = build_plan(batch=2, image=64, num_classes=10, fused=True, blocks=(1, 1, 1, 1))
        gpu = HotPathGPU(plan, communicator=None, world=1, seed=3, pool_argmax=flag)
        gpu.run_step()
        torch.cuda.synchronize()
        outs.append({p: gpu.t[p].clone() for p in plan["params"]})
        outs[-1]["bn1.dx"] = gpu.t["bn1.dx"].clone()
    for p in outs[0]:
        assert torch.equal(outs[0][p], outs[1][p]), p


def test_fused_and_unfused_plans_agree_bitwise():
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import build_plan
    outs = []
    for fused in (False, True):
        plan = build_plan(batch=2, image=64, num_classes=10, fused=fused, blocks=(1, 1, 1, 1))
        gpu = HotPathGPU(plan, communicator=None, world=1, seed=3)
        gpu.run_step()
        torch.cuda.synchronize()
        outs.append({p: gpu.t[p].clone() for p in plan["params"]})
    for p in outs[0]:
        assert torch.equal(outs[0][p], outs[1][p]), p


@pytest.mark.parametrize("which", ["mlp", "cnn"])
def test_small_config_steps_match_oracle(which):
    """The two small reference configurations: 1 (MLP 784-4096-4096-10, batch 256) and 2 (small CNN,
    batch 64) at their full sizes: one backward + SGD-momentum step, eager and
    fused, against the oracle executor."""
    from oracle.path import OraclePath
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import build_cnn_plan, build_mlp_plan, fuse_plan
    plan = build_mlp_plan() if which == "mlp" else build_cnn_plan()
    lr = 0.05 if which == "mlp" else 0.005
    wd = 0.0 if which == "mlp" else 1e-5
    for p in (plan, fuse_plan(plan)):
        gpu = HotPathGPU(p, communicator=None, world=1, seed=0, lr=lr, momentum=0.9, weight_decay=wd)
        host = gpu.host_copy()
        OraclePath(p, host, lr=lr, momentum=0.9, weight_decay=wd).run_step()
        gpu.run_step()
        torch.cuda.synchronize()
        got = gpu.host_copy()
        for name, spec in p["tensors"].items():
            if spec.kind == "grad":
                close(got[name], host[name], 2e-5, name)
        for name in p["params"]:
            close(got["d:" + name], host["d:" + name], 2e-5, "grad " + name)
            close(got[name], host[name], 1e-6, "param " + name)


@pytest.mark.parametrize("dist_option", ["plain", "half"])
def test_step_with_communicator_graph_and_update_on_arrival(dist_option):
    """One-rank communicator in the loop: bucketed synchronisation on the side
    streams, per-bucket SGD as each bucket lands, the whole step replayed from a
    CUDA graph.  Must equal the oracle's step (a one-rank all-reduce is the
    identity; fp16 transport rounds the gradients once)."""
    from oracle.path import OraclePath
    from singa_b200.communicator import Communicator, NcclIdHolder
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import build_plan, fuse_plan
    plan = fuse_plan(build_plan(batch=2, image=64, num_classes=10, blocks=(1, 1, 1, 1)))
    comm = Communicator(torch.cuda.current_device(), 1, NcclIdHolder(), buffSize=4194304)
    try:
        gpu = HotPathGPU(plan, communicator=comm, world=1, seed=9, dist_option=dist_option, threshold=20000)
        assert gpu.update_on_arrival and len(gpu.events) > 3
        host = gpu.host_copy()
        ref = OraclePath(plan, host, dist_option=dist_option)
        ref.run_step()
        ref.run_step()
        gpu.run_step()
        g = gpu.capture()
        g.replay()
        torch.cuda.synchronize()
        got = gpu.host_copy()
        tol = 2e-3 if dist_option == "half" else 1e-6
        for p in plan["params"]:
            close(got[p], host[p], tol, "param " + p)
        gpu.release_graph()
        del g
    finally:
        import gc
        gc.collect()
        torch.cuda.synchronize()
        comm.close()


@pytest.mark.parametrize("dist_option", ["plain", "half"])
def test_buckets_wait_for_the_kernels_that_produce_their_gradients(dist_option):
    """Every bucket's collective (and the update enqueued behind it on a side
    stream) must be ordered after the compute-stream kernels that wrote that
    bucket's gradients IN THIS STEP - for every bucket, not only the first.
    The step is built so that a missing edge cannot go unnoticed: the whole
    gradient arena is overwritten with a huge sentinel by the first kernel of
    the step, a slow elementwise kernel sits in front of every batch-norm
    backward call, and each stand-in weight gradient is written right before
    it is reported ready.  A collective or update that ran early would consume
    the sentinel.  Captured once, replayed with fresh labels each time;
    parameters must equal the oracle executor's after every replay."""
    from oracle.path import OraclePath
    from singa_b200.communicator import Communicator, NcclIdHolder
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import Op, Tensor, add_wgrad_refresh, build_plan, fuse_plan
    plan = fuse_plan(build_plan(batch=2, image=64, num_classes=10, blocks=(1, 1, 1, 1)))
    plan = add_wgrad_refresh(plan, where="each")
    T = dict(plan["tensors"])
    big = (64 * 1024 * 1024,)                                    # 256 MB per operand: ~0.1 ms per delay kernel
    for n in ("delay.a", "delay.b", "delay.out"):
        T[n] = Tensor(n, big, "grad")
    ops = [Op("fill", dict(x="grad_arena", value=3.0e30))]
    for op in plan["ops"]:
        if op.kind in ("bn_bwd", "bn_relu_bwd"):
            ops.append(Op("add_out", dict(a="delay.a", b="delay.b", out="delay.out")))
        ops.append(op)
    plan = dict(plan, ops=ops, tensors=T)
    comm = Communicator(torch.cuda.current_device(), 1, NcclIdHolder(), buffSize=4194304)
    try:
        gpu = HotPathGPU(plan, communicator=comm, world=1, seed=11, dist_option=dist_option, threshold=2000)
        assert gpu.update_on_arrival
        assert sum(1 for k, _ in gpu.events if k == "fused") >= 4 and len(gpu.events) >= 20
        host = gpu.host_copy()
        for n in ("delay.a", "delay.b", "delay.out"):
            host.pop(n)                                          # the checker has no use for the delay operands
        ref_plan = dict(plan, ops=[o for o in plan["ops"] if not (o.kind == "add_out" and o.args["a"] == "delay.a")])
        ref = OraclePath(ref_plan, host, dist_option=dist_option)
        tol = 2e-3 if dist_option == "half" else 1e-6
        rng = np.random.default_rng(5)

        def new_labels():
            lab = rng.integers(0, 10, host["labels"].shape).astype(np.int32)
            host["labels"][...] = lab
            gpu.t["labels"].copy_(torch.from_numpy(lab))

        def check(what):
            torch.cuda.synchronize()
            got = gpu.host_copy()
            for p in plan["params"]:
                assert np.isfinite(got[p]).all(), "%s: %s consumed the sentinel" % (what, p)
                close(got[p], host[p], tol, "%s: param %s" % (what, p))

        ref.run_step()
        gpu.run_step()
        check("eager step")
        g = gpu.capture()
        for k in range(3):
            new_labels()
            ref.run_step()
            g.replay()
            check("replay %d" % k)
        gpu.release_graph()
        del g
    finally:
        import gc
        gc.collect()
        torch.cuda.synchronize()
        comm.close()


def test_refreshed_stand_in_gradients_do_not_compound():
    """The weight gradients of the contractions are rewritten from pristine
    copies every step, so repeated steps update with the same finite values
    (an in-place all-reduce would otherwise scale a never-rewritten gradient
    by the world size on every step)."""
    from oracle.path import OraclePath
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import add_wgrad_refresh, build_plan, fuse_plan
    plan = add_wgrad_refresh(fuse_plan(build_plan(batch=2, image=64, num_classes=10, blocks=(1, 1, 1, 1))))
    assert plan["ops"][0].kind == "wgrad_refresh" and len(plan["ops"][0].args["params"]) > 10
    gpu = HotPathGPU(plan, communicator=None, world=1, seed=2)
    host = gpu.host_copy()
    ref = OraclePath(plan, host)
    gpu.t["d:conv1.W"].fill_(7.0)                 # whatever the last step left is overwritten
    for _ in range(2):
        ref.run_step()
        gpu.run_step()
    torch.cuda.synchronize()
    got = gpu.host_copy()
    assert np.array_equal(got["d:conv1.W"], got["wsyn:conv1.W"])
    for p in plan["params"]:
        close(got[p], host[p], 1e-6, "param " + p)


def test_relu_bit_record_gives_the_same_step_bitwise():
    """The ReLU forward partner's one-bit-per-element record instead of the
    stored ReLU input, in all three consumers (ReLU backward alone, joined,
    folded into batch-norm backward): same parameters bit for bit, and the
    step still equals the oracle executor's."""
    from oracle.path import OraclePath
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import build_plan, fuse_plan, mask_plan
    outs = []
    for masked in (False, True):
        plan = fuse_plan(build_plan(batch=2, image=64, num_classes=10, blocks=(2, 1, 1, 1)))
        if masked:
            plan = mask_plan(plan)
            kinds = [o.kind for o in plan["ops"]]
            assert "bn_relu_mask_bwd" in kinds and "add_relu_mask_bwd" in kinds and "relu_mask_bwd" in kinds
            assert not any(k in kinds for k in ("bn_relu_bwd", "add_relu_bwd", "relu_bwd"))
        gpu = HotPathGPU(plan, communicator=None, world=1, seed=3)
        if masked:
            host = gpu.host_copy()
            OraclePath(plan, host).run_step()
        gpu.run_step()
        torch.cuda.synchronize()
        outs.append({p: gpu.t[p].clone() for p in plan["params"]})
        outs[-1]["bn1.dx"] = gpu.t["bn1.dx"].clone()
    for p in outs[0]:
        assert torch.equal(outs[0][p], outs[1][p]), p
    got = gpu.host_copy()
    for p in plan["params"]:
        close(got[p], host[p], 1e-6, "param " + p)


@pytest.mark.parametrize("n", [1, 3, 31, 32, 33, 4096, 100003])
def test_relu_forward_record_layout(n):
    """y = max(x, 0); bit i of the record = x[i] > 0 in plain element order,
    for aligned and misaligned buffers and every tail length."""
    from singa_b200 import _lib
    L = _lib.lib()
    for shift in (0, 1):
        buf = torch.randn(n + 8, device="cuda")
        buf[::3] = 0.0
        x = buf[shift:shift + n]
        ybuf = torch.empty(n + 8, device="cuda")
        y = ybuf[shift:shift + n]
        rec = torch.full((L.sgb_relu_mask_bytes(n),), 0xFF, dtype=torch.uint8, device="cuda")
        _lib.call("sgb_relu_forward_mask_f32", x.data_ptr(), y.data_ptr(), rec.data_ptr(), n,
                  torch.cuda.current_stream().cuda_stream)
        dy = torch.randn(n + 8, device="cuda")[shift:shift + n]
        dx = torch.empty(n + 8, device="cuda")[shift:shift + n]
        _lib.call("sgb_relu_backward_mask_f32", dy.data_ptr(), rec.data_ptr(), dx.data_ptr(), n,
                  torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(y, torch.relu(x))
        bits = np.unpackbits(rec.cpu().numpy(), bitorder="little")[:n]
        assert np.array_equal(bits.astype(bool), (x > 0).cpu().numpy())
        assert torch.equal(dx, torch.where(x > 0, dy, torch.zeros_like(dy)))
