"""Multi-process communicator check, launched by tests/test_comm_gpu.py as
``python -m torch.distributed.run --nproc-per-node N tests/dist_worker.py``.
One rank per GPU.  The NCCL id travels over a gloo process group; every rank
re-creates all ranks' seeded inputs, so the oracle's result is known locally."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import comm as ocomm          # noqa: E402  (checker)
from singa_b200 import _lib, opt          # noqa: E402
from singa_b200.communicator import Communicator, NcclIdHolder   # noqa: E402


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, want, rtol, what):
    want = np.asarray(want, np.float64)
    err = np.abs(np.asarray(got, np.float64) - want).max()
    scale = max(np.abs(want).max(), 1e-30)
    assert err <= rtol * scale, "%s: rel err %.3e" % (what, err / scale)


def main():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(local)
    box = [NcclIdHolder().id if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(local, world, NcclIdHolder(box[0]), buffSize=4194304)
    assert comm.world_size == world and comm.global_rank == rank

    # (a) the reference's own distributed test: grad = 1, param = 10 -> 9.9
    sgd = opt.SGD(lr=0.1)
    modes = {
        "all_reduce": lambda g: comm.synch(g),
        "fused_all_reduce": lambda g: (comm.fusedSynch([g], False), comm.fusedSynch([g], True)),
        "all_reduce_half": lambda g: comm.synchHalf(g),
        "fused_all_reduce_half": lambda g: (comm.fusedSynchHalf([g], False), comm.fusedSynchHalf([g], True)),
        "sparse_threshold": lambda g: comm.sparsification(g, None, 0.05, False),
        "sparse_topk": lambda g: comm.sparsification(g, None, 1.0, True),
    }
    for name, fn in modes.items():
        param = torch.full((10, 10), 10.0, device="cuda")
        grad = torch.full((10, 10), 1.0, device="cuda")
        fn(grad)
        comm.wait()
        sgd.apply(name, param, grad, grad_scale=float(np.float32(1.0) / np.float32(world)))
        np.testing.assert_array_almost_equal(param.cpu().numpy(), 10 - 0.1, decimal=5, err_msg=name)

    # (b) + (c) seeded random gradients through the DistOpt bucket policy
    sizes = [1000, 2048000, 2048, 2048, 1048576, 2359296, 512, 512, 1048576, 262144, 64, 64, 9408]
    def grads_of(r, step):
        rng = np.random.default_rng(1000 * step + r)
        return [(rng.standard_normal(n) * 1e-2).astype(np.float32) for n in sizes]
    for half in (False, True):
        allg = [grads_of(r, 1) for r in range(world)]
        mine = [dev(a) for a in allg[rank]]
        plist, glist, acc = [], [], 0
        direct = comm.synchHalf if half else comm.synch
        fused = comm.fusedSynchHalf if half else comm.fusedSynch
        for g in mine:                                   # opt.py:846-862
            if g.numel() > 2097152:
                direct(g)
            else:
                glist.append(g)
                fused([g], False)
                acc += g.numel()
                if acc > 2097152:
                    fused(glist, True)
                    acc, glist = 0, []
        if glist:
            fused(glist, True)
        comm.wait()
        torch.cuda.synchronize()
        for i, g in enumerate(mine):
            per_rank = [allg[r][i] for r in range(world)]
            want = ocomm.allreduce_half(per_rank) if half else ocomm.allreduce_sum(per_rank)
            close(g.cpu().numpy(), want, 1e-3 if half else 1e-5, "%s tensor %d" % ("half" if half else "fp32", i))

    # (d) + (e) sparsified sync with residuals over three steps: bit-exact
    n = 300007
    for topk, spars, mode in ((False, 2e-3, None), (True, 0.01, "magnitude"), (True, 0.01, "compat"),
                              (True, 0.3, "compat")):
        if mode:
            comm.set_topk_mode(mode)
        scale = 3.0 if (mode == "compat" and spars == 0.3) else 1e-3
        accs = [np.zeros(n, np.float32) for _ in range(world)]
        d_acc = torch.zeros(n, device="cuda")
        for step in range(3):
            gs = [(np.random.default_rng(20 * r + step).standard_normal(n) * scale).astype(np.float32)
                  for r in range(world)]
            g = dev(gs[rank])
            # step 0: one tensor; step 1: two tensors back to back (exchanged in place);
            # step 2: two tensors apart in memory (copied through the communicator's buffers)
            if step == 1:
                parts = [g[:100001], g[100001:]]
            elif step == 2:
                parts = [g[:100001].clone(), g[100001:].clone()]
            else:
                parts = [g]
            comm.fusedSparsification(parts, d_acc, spars, topk)
            comm.wait()
            torch.cuda.synchronize()
            if step == 2:
                g = torch.cat(parts)
            if topk:
                dense, accs, _ = ocomm.sparse_topk_step(gs, accs, spars, mode)
            else:
                dense, accs, _ = ocomm.sparse_threshold_step(gs, accs, spars)
            assert np.array_equal(g.cpu().numpy().view(np.uint32), dense.view(np.uint32)), \
                ("dense", topk, mode, step)
            assert np.array_equal(d_acc.cpu().numpy().view(np.uint32), accs[rank].view(np.uint32)), \
                ("residual", topk, mode, step)

    # (e2) the capacity-bounded threshold exchange (no host wait for the counts)
    thr = 2e-3
    # ample capacity: bit for bit the reference's exchange, over three steps with residuals
    accs = [np.zeros(n, np.float32) for _ in range(world)]
    d_acc = torch.zeros(n, device="cuda")
    for step in range(3):
        gs = [(np.random.default_rng(500 + 20 * r + step).standard_normal(n) * 1e-3).astype(np.float32)
              for r in range(world)]
        g = dev(gs[rank])
        comm.boundedSparsification([g], d_acc, thr, n)
        comm.wait()
        torch.cuda.synchronize()
        dense, accs, _ = ocomm.sparse_threshold_step(gs, accs, thr)
        assert np.array_equal(g.cpu().numpy().view(np.uint32), dense.view(np.uint32)), ("bounded dense", step)
        assert np.array_equal(d_acc.cpu().numpy().view(np.uint32), accs[rank].view(np.uint32)), ("bounded acc", step)
    assert comm.sparseDropped() == 0
    # tight capacity over two steps: every rank sends its first `cap` selections (index order), the others
    # stay in the residual and compete again in the next step
    cap = 1000
    accs = [np.zeros(n, np.float32) for _ in range(world)]
    d_acc = torch.zeros(n, device="cuda")
    total_held = 0
    for step in range(2):
        gs = [(np.random.default_rng(900 + 20 * r + step).standard_normal(n) * 1e-3).astype(np.float32)
              for r in range(world)]
        g = dev(gs[rank])
        comm.boundedSparsification([g], d_acc, thr, cap)
        comm.wait()
        torch.cuda.synchronize()
        dense, accs, held = ocomm.sparse_threshold_bounded_step(gs, accs, thr, cap)
        assert held[rank] > 0
        total_held += held[rank]
        assert np.array_equal(g.cpu().numpy().view(np.uint32), dense.view(np.uint32)), ("tight dense", step)
        assert np.array_equal(d_acc.cpu().numpy().view(np.uint32), accs[rank].view(np.uint32)), ("tight acc", step)
    assert comm.sparseDropped() == total_held, (comm.sparseDropped(), total_held)
    # inside a captured graph: two replays with fresh gradients equal two eager calls
    side = torch.cuda.Stream()
    g_buf, acc_buf = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    fresh = [dev((np.random.default_rng(1300 + 10 * k + rank).standard_normal(n) * 1e-3).astype(np.float32))
             for k in range(2)]
    with torch.cuda.stream(side):
        comm.boundedSparsification([g_buf], acc_buf, thr, n)   # warm-up outside capture
        comm.wait()
        side.synchronize()
        acc_buf.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            comm.boundedSparsification([g_buf], acc_buf, thr, n)
            comm.wait()
    torch.cuda.synchronize()
    e_acc = torch.zeros(n, device="cuda")
    for k in range(2):
        g_buf.copy_(fresh[k])
        graph.replay()
        torch.cuda.synchronize()
        e_g = fresh[k].clone()
        comm.boundedSparsification([e_g], e_acc, thr, n)
        comm.wait()
        torch.cuda.synchronize()
        assert torch.equal(g_buf, e_g) and torch.equal(acc_buf, e_acc), ("graph replay", k)
    del graph

    # (g) DistOpt.backward_and_partial_update through the real communicator:
    # local SGD-momentum updates, then one partition of the parameters averaged
    from oracle import cpu as ocpu
    psizes = [1000, 2048000, 2048, 2048, 1048576, 2359296, 512, 64, 2400000, 9408]
    plan = ocomm.plan_buckets(psizes)

    def pgrads(r, step):
        rng = np.random.default_rng(7000 + 10 * step + r)
        return [(rng.standard_normal(k) * 1e-2).astype(np.float32) for k in psizes]
    dopt = opt.DistOpt(opt.SGD(lr=0.1, momentum=0.9), communicator=comm)
    params = [torch.zeros(k, device="cuda") for k in psizes]
    want = [[np.zeros(k, np.float32) for k in psizes] for _ in range(world)]
    mom = [[np.zeros(k, np.float32) for k in psizes] for _ in range(world)]
    for step in range(len(plan) + 1):
        mine = [dev(a) for a in pgrads(rank, step)]
        dopt.backward_and_partial_update((("q%d" % i, p_, g_) for i, (p_, g_) in enumerate(zip(params, mine))))
        for r in range(world):
            for i, g_ in enumerate(pgrads(r, step)):
                ocpu.sgd_update(want[r][i], g_.copy(), mom[r][i], 0.1, momentum=0.9)
        for i in plan[step % len(plan)][1]:
            avg = ocomm.divide_by_world(ocomm.allreduce_sum([want[r][i] for r in range(world)]), world)
            for r in range(world):
                want[r][i][...] = avg
    torch.cuda.synchronize()
    for i, p_ in enumerate(params):
        close(p_.cpu().numpy(), want[rank][i], 1e-5, "partial update, parameter %d" % i)

    # (f) host-side failure injection: a bucket that overflows is refused, not written
    big = torch.zeros(4194304, device="cuda")
    comm.fusedSynch([big], False)
    try:
        comm.fusedSynch([torch.zeros(8, device="cuda")], False)
        raise AssertionError("overflow was accepted")
    except _lib.SgbError as e:
        assert e.status == -8
    comm.fusedSynch([big], True)
    comm.wait()
    torch.cuda.synchronize()
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d of %d: communicator checks passed" % (rank, world))


if __name__ == "__main__":
    main()
