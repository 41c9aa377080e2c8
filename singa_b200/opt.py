"""SGD and DistOpt drivers with the reference's structure (python/singa/opt.py),
written against ``singa_b200.singa_wrap`` / ``singa_b200.communicator``.

The reference builds gradients with its autograd generator; this module takes
any iterable of ``(param, grad)`` pairs in the order gradients are produced
(what ``autograd.backward(loss)`` yields, python/singa/autograd.py:128-224).
"""
import numpy as np

from . import singa_wrap as sw


def plan_buckets(sizes, threshold=2097152):
    """Bucket policy of DistOpt.backward_and_update (opt.py:846-862): a tensor
    larger than ``threshold`` is reduced directly; smaller ones are staged and
    the bucket is flushed as soon as it holds more than ``threshold``
    elements.  Returns [("direct" | "fused", [indices])] in issue order."""
    events, glist, acc = [], [], 0
    for i, n in enumerate(sizes):
        if n > threshold:
            events.append(("direct", [i]))
            continue
        glist.append(i)
        acc += n
        if acc > threshold:
            events.append(("fused", glist))
            glist, acc = [], 0
    if glist:
        events.append(("fused", glist))
    return events


class SGD(object):
    """SGD with momentum / dampening / weight decay / Nesterov (opt.py:161-333).

    ``apply`` is one fused kernel pass per call; ``apply_many`` updates a whole
    parameter list in one launch group.  Hyper-parameters are python floats
    (the reference keeps them in one-element device tensors)."""

    def __init__(self, lr=0.1, momentum=0, dampening=0, weight_decay=0, nesterov=False):
        if momentum < 0.0:
            raise ValueError("Invalid momentum value: {}".format(momentum))
        if weight_decay < 0.0:
            raise ValueError("Invalid weight_decay value: {}".format(weight_decay))
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        self.lr, self.momentum, self.dampening = lr, momentum, dampening
        self.weight_decay, self.nesterov = weight_decay, nesterov
        self.moments = dict()
        self.step_counter = 0

    def _moment(self, name, like):
        import torch
        if name not in self.moments:
            self.moments[name] = torch.zeros_like(like)
        return self.moments[name]

    def apply(self, param_name, param_value, param_grad, grad_scale=1.0):
        assert param_value.shape == param_grad.shape, ("shape mismatch", param_value.shape,
                                                       param_grad.shape)
        self.apply_many([param_name], [param_value], [param_grad], grad_scale)

    def apply_many(self, names, params, grads, grad_scale=1.0):
        moments = [self._moment(n, p) for n, p in zip(names, params)] if self.momentum != 0 else None
        sw.sgd_update_multi(params, grads, moments, self.lr, self.momentum, self.dampening,
                            self.weight_decay, self.nesterov, grad_scale)

    def step(self):
        self.step_counter += 1


class DistOpt(object):
    """Data-parallel wrapper of an optimizer (opt.py:686-1094).

    ``nccl_id`` is a ``communicator.NcclIdHolder`` shared by all ranks.  The
    1/world scaling of ``DistOpt.update`` (opt.py:738-746) and the optimizer
    step run as ONE multi-tensor launch group at the end of each
    ``backward_and_*`` call (``grad_scale`` of the fused SGD kernel)."""

    def __init__(self, opt, nccl_id=None, local_rank=0, world_size=1, buffSize=4194304,
                 communicator=None):
        self.opt = opt
        if communicator is None:
            from .communicator import Communicator
            communicator = Communicator(local_rank, world_size, nccl_id, buffSize)
        # any object with the reference Communicator's methods and rank fields
        self.communicator = communicator
        self.world_size = self.communicator.world_size
        self.local_rank = self.communicator.local_rank
        self.global_rank = self.communicator.global_rank

    # thin forwards, names as in the reference
    def all_reduce(self, tensor):
        self.communicator.synch(tensor)

    def fused_all_reduce(self, tensors, send=True):
        self.communicator.fusedSynch(tensors, send)

    def all_reduce_half(self, tensor):
        self.communicator.synchHalf(tensor)

    def fused_all_reduce_half(self, tensors, send=True):
        self.communicator.fusedSynchHalf(tensors, send)

    def sparsification(self, tensor, accumulation, spars, topK):
        self.communicator.sparsification(tensor, accumulation, spars, topK)

    def fused_sparsification(self, tensors, accumulation, spars, topK):
        self.communicator.fusedSparsification(tensors, accumulation, spars, topK)

    def wait(self):
        self.communicator.wait()

    def update(self, param, grad, name=None):
        """grad /= world_size, then the wrapped optimizer's update."""
        scale = float(np.float32(1.0) / np.float32(self.world_size))
        self.opt.apply(name if name is not None else id(param), param, grad, grad_scale=scale)

    def _update_all(self, plist):
        scale = float(np.float32(1.0) / np.float32(self.world_size))
        names = [n for n, _, _ in plist]
        self.opt.apply_many(names, [p for _, p, _ in plist], [g for _, _, g in plist], scale)
        self.opt.step()

    def _sync_dense(self, grad_stream, threshold, direct, fused):
        plist, glist, acc = [], [], 0
        for name, p, g in grad_stream:
            if g.numel() > threshold:
                direct(g)
            else:
                glist.append(g)
                fused([g], False)
                acc += g.numel()
                if acc > threshold:
                    fused(glist, True)
                    acc, glist = 0, []
            plist.append((name, p, g))
        if glist:
            fused(glist, True)
        self.wait()
        return plist

    def backward_and_update(self, grad_stream, threshold=2097152):
        """opt.py:826-865 over (name, param, grad) triples."""
        self._update_all(self._sync_dense(grad_stream, threshold, self.all_reduce,
                                          self.fused_all_reduce))

    def backward_and_update_half(self, grad_stream, threshold=2097152, clipping=False,
                                 clip_Value=100):
        """opt.py:867-920: fp16 transport of fp32 gradients."""
        def clipped(stream):
            for name, p, g in stream:
                if clipping:
                    sw.Clamp(g, -clip_Value, clip_Value, out=g)
                yield name, p, g
        self._update_all(self._sync_dense(clipped(grad_stream), threshold, self.all_reduce_half,
                                          self.fused_all_reduce_half))

    def _divide_by_world(self, t):
        sw.DivFloatWithRet(t, self.world_size, t)

    def backward_and_partial_update(self, grad_stream, threshold=2097152):
        """opt.py:922-992 (asynchronous variant): every parameter is updated with
        its LOCAL gradient first; then ONE partition of the PARAMETERS - the
        ``self.partial``-th bucket in production order, cycling - is all-reduced
        and averaged.  A partition is a tensor above ``threshold`` or a bucket of
        smaller ones, exactly as in ``backward_and_update``."""
        self.partial = getattr(self, "partial", 0) + 1
        names, params, grads = [], [], []
        k, acc, bucket, reduced = 0, 0, [], []
        picked = []                                   # (kind, tensors) of the partition to exchange
        for name, p, g in grad_stream:
            names.append(name)
            params.append(p)
            grads.append(g)
            if p.numel() > threshold:
                k += 1
                if k == self.partial:
                    picked.append(("direct", [p]))
            else:
                bucket.append(p)
                acc += p.numel()
                if acc > threshold:
                    k += 1
                    if k == self.partial:
                        picked.append(("fused", bucket))
                    acc, bucket = 0, []
        if bucket:
            k += 1
            if k == self.partial:
                picked.append(("fused", bucket))
        # local update of everything (grad_scale 1: no averaging of gradients in this mode)
        self.opt.apply_many(names, params, grads, 1.0)
        for kind, tensors in picked:
            if kind == "direct":
                self.all_reduce(tensors[0])
            else:
                self.fused_all_reduce(tensors, send=False)
                self.fused_all_reduce(tensors)
            reduced = tensors
        self.wait()
        for r in reduced:
            self._divide_by_world(r)                   # "r /= world_size" on the exchanged parameters
        if k == self.partial:
            self.partial = 0
        self.opt.step()

    def backward_and_sparse_update(self, grad_stream, threshold=2097152, spars=0.05, topK=False,
                                   corr=True):
        """opt.py:994-1094: sparsified synchronisation with local residuals."""
        import torch
        if not hasattr(self, "sparsInit") and corr:
            self.gradAccumulation = []
            self.sparsInit = False
        plist, glist, acc, k = [], [], 0, -1

        def residual(n, like):
            if corr and not self.sparsInit:
                self.gradAccumulation.append(torch.zeros(n, dtype=like.dtype, device=like.device))
            return self.gradAccumulation[k] if corr else None

        for name, p, g in grad_stream:
            if g.numel() > threshold:
                k += 1
                self.sparsification(g, residual(g.numel(), g), spars, topK)
            else:
                glist.append(g)
                acc += g.numel()
                if acc > threshold:
                    k += 1
                    self.fused_sparsification(glist, residual(acc, g), spars, topK)
                    acc, glist = 0, []
            plist.append((name, p, g))
        if glist:
            k += 1
            self.fused_sparsification(glist, residual(acc, glist[0]), spars, topK)
        self.wait()
        self.sparsInit = True
        self._update_all(plist)
