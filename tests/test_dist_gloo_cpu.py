"""World-size-2 check of the host-side data-parallel logic on CPU (gloo): the
DistOpt driver (bucket policy, staging/flush order, 1/world scaling, optimizer
step) runs in two processes against a communicator double that moves the data
with gloo and an optimizer double that uses the oracle's SGD.  The result must
equal a single-process simulation of both ranks."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIZES = [1000, 2048000, 2048, 2048, 1048576, 2359296, 512, 512, 600000, 64, 2400000, 9408]


def grads_of(rank, step):
    rng = np.random.default_rng(100 * step + rank)
    return [(rng.standard_normal(n) * 1e-2).astype(np.float32) for n in SIZES]


class GlooCommunicator(object):
    """Same method names and call protocol as singa_b200.communicator.Communicator."""

    def __init__(self, rank, world, buffSize):
        self.global_rank = self.local_rank = rank
        self.world_size = world
        self.buff = buffSize
        self.staged = 0
        self.log = []

    def synch(self, t):
        self.log.append(("synch", t.numel()))
        dist.all_reduce(t)

    def fusedSynch(self, ts, send=True):
        if not send:
            n = sum(t.numel() for t in ts)
            assert self.staged + n <= self.buff, "bucket overflow"
            self.staged += n
            self.log.append(("stage", n))
            return
        assert self.staged == sum(t.numel() for t in ts), "flush list must equal what was staged"
        flat = torch.cat([t.reshape(-1) for t in ts])
        dist.all_reduce(flat)
        off = 0
        for t in ts:
            t.copy_(flat[off:off + t.numel()].view_as(t))
            off += t.numel()
        self.log.append(("flush", self.staged))
        self.staged = 0

    def wait(self):
        self.log.append(("wait", 0))


class OracleSGD(object):
    def __init__(self, lr, momentum):
        self.lr, self.momentum, self.moments, self.steps = lr, momentum, {}, 0

    def apply_many(self, names, params, grads, grad_scale=1.0):
        from oracle import cpu
        for n, p, g in zip(names, params, grads):
            m = self.moments.setdefault(n, np.zeros(p.numel(), np.float32))
            gg = (g.numpy().ravel() * np.float32(grad_scale)).astype(np.float32)
            pv = p.numpy().ravel()
            cpu.sgd_update(pv, gg, m, self.lr, momentum=self.momentum)

    def step(self):
        self.steps += 1


def worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from singa_b200.opt import DistOpt, plan_buckets
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    comm = GlooCommunicator(rank, world, 4194304)
    opt = DistOpt(OracleSGD(0.1, 0.9), communicator=comm)
    params = [torch.zeros(n) for n in SIZES]
    for step in range(2):
        grads = [torch.from_numpy(g) for g in grads_of(rank, step)]
        opt.backward_and_update((("p%d" % i, p, g) for i, (p, g) in enumerate(zip(params, grads))))
    # the issue order follows the bucket plan
    plan = plan_buckets(SIZES)
    assert sum(1 for k, _ in comm.log if k == "flush") == 2 * sum(1 for k, _ in plan if k == "fused")
    assert sum(1 for k, _ in comm.log if k == "synch") == 2 * sum(1 for k, _ in plan if k == "direct")
    assert opt.opt.steps == 2
    out[rank] = [p.numpy().copy() for p in params]
    dist.barrier()
    dist.destroy_process_group()


def partial_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from singa_b200.opt import DistOpt, plan_buckets

    class HostDistOpt(DistOpt):
        def _divide_by_world(self, t):                 # the product scales on the GPU; same fp32 product here
            t.mul_(float(np.float32(1.0) / np.float32(self.world_size)))

    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    comm = GlooCommunicator(rank, world, 4194304)
    opt = HostDistOpt(OracleSGD(0.1, 0.9), communicator=comm)
    params = [torch.zeros(n) for n in SIZES]
    nparts = len(plan_buckets(SIZES))
    for step in range(nparts + 2):                     # one full cycle of partitions and a bit more
        grads = [torch.from_numpy(g) for g in grads_of(rank, step)]
        opt.backward_and_partial_update((("p%d" % i, p, g) for i, (p, g) in enumerate(zip(params, grads))))
        assert opt.partial == (step + 1) % nparts
    exchanges = sum(1 for k, _ in comm.log if k in ("flush", "synch"))
    assert exchanges == nparts + 2                     # exactly one partition per step
    out[rank] = [p.numpy().copy() for p in params]
    dist.barrier()
    dist.destroy_process_group()


def test_partial_update_two_ranks_over_gloo():
    """backward_and_partial_update: local updates everywhere, then one partition
    of the PARAMETERS (cycling through the bucket plan) is summed over the ranks
    and divided by the world size."""
    from oracle import comm as ocomm, cpu
    world = 2
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(partial_worker, args=(world, free_port(), out), nprocs=world, join=True)
    plan = ocomm.plan_buckets(SIZES)
    params = [[np.zeros(n, np.float32) for n in SIZES] for _ in range(world)]
    moments = [[np.zeros(n, np.float32) for n in SIZES] for _ in range(world)]
    for step in range(len(plan) + 2):
        for r in range(world):
            for i, g in enumerate(grads_of(r, step)):
                cpu.sgd_update(params[r][i], g.copy(), moments[r][i], 0.1, momentum=0.9)
        _, members = plan[step % len(plan)]
        for i in members:
            avg = ocomm.divide_by_world(params[0][i] + params[1][i], world)
            for r in range(world):
                params[r][i][...] = avg
    for r in range(world):
        for got, want in zip(out[r], params[r]):
            assert np.array_equal(got, want)


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_distopt_host_logic_two_ranks_over_gloo():
    from oracle import comm as ocomm, cpu
    world = 2
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(worker, args=(world, free_port(), out), nprocs=world, join=True)
    # single-process simulation of both ranks
    params = [np.zeros(n, np.float32) for n in SIZES]
    moments = [np.zeros(n, np.float32) for n in SIZES]
    for step in range(2):
        per_rank = [grads_of(r, step) for r in range(world)]
        for i in range(len(SIZES)):
            total = per_rank[0][i] + per_rank[1][i]          # gloo sums two fp32 values: exact order-free
            g = ocomm.divide_by_world(total, world)
            cpu.sgd_update(params[i], g.copy(), moments[i], 0.1, momentum=0.9)
    for r in range(world):
        for got, want in zip(out[r], params):
            assert np.array_equal(got, want)
