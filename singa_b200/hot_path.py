"""GPU executor of a hot-path plan (see ``resnet50_path.build_plan``).

Owns the device tensors (torch is the allocator), turns every op into one
pre-bound C-ABI call, replays DistOpt's bucket policy on the communicator as
gradients become ready, and finishes with the fused multi-tensor SGD update.
The whole step can be captured once into a CUDA graph and replayed, which is
this implementation's counterpart of the reference's buffered-operation graph
(``Device::EnableGraph`` / ``RunGraph``).
"""
import ctypes as C

import numpy as np
import torch

from . import _lib
from .opt import plan_buckets
from .resnet50_path import numel


def _table(tensors):
    n = len(tensors)
    return ((C.c_void_p * n)(*[t.data_ptr() for t in tensors]),
            (C.c_size_t * n)(*[t.numel() for t in tensors]), n)


class HotPathGPU(object):
    def __init__(self, plan, communicator=None, world=1, seed=0, lr=0.1, momentum=0.9,
                 weight_decay=1e-5, threshold=2097152, dist_option="plain", spars=0.05,
                 device=None, update_on_arrival=True, pool_argmax=False):
        self.plan, self.comm, self.world = plan, communicator, world
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.threshold, self.dist_option, self.spars = threshold, dist_option, spars
        # With a communicator, every bucket's parameters are updated on the
        # communicator's side stream as soon as that bucket's reduced gradients
        # have landed, overlapped with the rest of the backward pass (same
        # results as updating everything after the final wait).
        self.update_on_arrival = bool(update_on_arrival) and communicator is not None \
            and dist_option in ("plain", "half")
        # pool_argmax: max-pool backward consumes the arg-max record of the forward
        # partner (produced once at set-up: the forward pass is outside this path)
        # instead of recomputing the winners from x and y.  Same dx bit for bit.
        self.pool_argmax = bool(pool_argmax)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.lib = _lib.lib()
        self.t = {}
        self._alloc(seed)
        self._bind()
        self.graph = None
        self.launches_per_step = None
        self.profile = False      # True: mark "bucket_ready" on the compute stream (communicator timing on)

    # ------------------------------------------------------------------ tensors
    def _alloc(self, seed):
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        T, dev = self.plan["tensors"], self.device

        def randn(shape, std=1.0, mean=0.0):
            return torch.randn(shape, generator=gen, device=dev) * std + mean

        # Parameter gradients live back to back, in the order they are produced,
        # in one arena: every bucket of the synchronisation policy is then a
        # contiguous slice and is all-reduced in place (no pack / unpack pass).
        names = self.plan["grad_order"]
        sizes = [numel(T["d:" + n].shape) for n in names]
        order = [names[i] for _, idx in plan_buckets(sizes, self.threshold) for i in idx]   # bucket by bucket
        total = sum(sizes)
        self.grad_arena = torch.empty(total, device=dev)
        arena_view, off = {}, 0
        for n in order:
            cnt = numel(T["d:" + n].shape)
            arena_view["d:" + n] = self.grad_arena[off:off + cnt].view(T["d:" + n].shape)
            off += cnt
        self.t["grad_arena"] = self.grad_arena
        # pristine stand-ins of the contractions' weight gradients, back to back in
        # refresh order (one flat buffer: a refresh is one multi-tensor copy)
        wsyn = [n for n, spec in T.items() if spec.kind == "wsyn"]
        self.wsyn_flat = torch.empty(sum(numel(T[n].shape) for n in wsyn), device=dev)
        self.wsyn_off, off = {}, 0
        for n in wsyn:
            cnt = numel(T[n].shape)
            self.wsyn_off[n] = off
            self.t[n] = self.wsyn_flat[off:off + cnt].view(T[n].shape)
            self.t[n].copy_(randn(T[n].shape, 1e-3))
            off += cnt
        for name, spec in T.items():
            k = spec.kind
            if k in ("wsyn", "mask"):
                continue
            if k == "pgrad" and name in arena_view:
                self.t[name] = arena_view[name]
                self.t[name].copy_(randn(spec.shape, 1e-3))
                continue
            if k == "label":
                self.t[name] = torch.randint(0, T["logits"].shape[1], spec.shape, generator=gen,
                                             device=dev, dtype=torch.int32)
            elif k == "act":
                self.t[name] = randn(spec.shape, 1.5, 0.2) if name.endswith(".x") and ".bn" in name or name == "bn1.x" \
                    else randn(spec.shape)
            elif k == "syn":
                self.t[name] = randn(spec.shape, 1e-2)
            elif k == "param":
                if name.endswith(".scale"):
                    self.t[name] = torch.ones(spec.shape, device=dev)
                elif name.endswith(".bias") or name == "fc.b":
                    self.t[name] = torch.zeros(spec.shape, device=dev)
                else:
                    self.t[name] = randn(spec.shape, 0.05)
            elif k == "pgrad":
                self.t[name] = randn(spec.shape, 1e-3)
            else:
                self.t[name] = torch.zeros(spec.shape, device=dev)
        # forward-consistent statistics and ReLU inputs (set-up only, not timed)
        for name in list(T):
            if name.endswith(".mean"):
                base = name[:-5]
                x = self.t[base + ".x"]
                var, mean = torch.var_mean(x, dim=(0, 2, 3), unbiased=False)
                self.t[base + ".mean"].copy_(mean)
                self.t[base + ".invstd"].copy_(torch.rsqrt(var))
                relu_name = {"bn1": "relu.x"}.get(base, base.replace(".bn", ".relu") + ".x")
                if relu_name in self.t and ".down" not in base and not base.endswith("bn3"):
                    s = self.t[base + ".scale"].view(1, -1, 1, 1)
                    b = self.t[base + ".bias"].view(1, -1, 1, 1)
                    self.t[relu_name].copy_((x - mean.view(1, -1, 1, 1)) * torch.rsqrt(var).view(1, -1, 1, 1) * s + b)
        if "maxpool.x" in self.t:
            self.t["maxpool.x"].copy_(torch.relu(self.t["relu.x"]))
            self.t["maxpool.y"].copy_(torch.nn.functional.max_pool2d(self.t["maxpool.x"], 3, 2, 1))
        for op in self.plan["ops"]:        # other max-pool layers: post-ReLU input, consistent output
            if op.kind == "maxpool_bwd" and op.args["x"] != "maxpool.x":
                a = op.args
                self.t[a["x"]].copy_(torch.relu(self.t[a["x"]]))
                self.t[a["y"]].copy_(torch.nn.functional.max_pool2d(self.t[a["x"]], a["kernel"], a["stride"], a["pad"]))
        # bit records of the ReLU forward partner (produced once at set-up: the
        # forward pass is outside this path), from the stored ReLU inputs
        for name, spec in T.items():
            if spec.kind != "mask":
                continue
            src = self.t[name[len("mask:"):]]
            n = src.numel()
            rec = torch.zeros(self.lib.sgb_relu_mask_bytes(n), dtype=torch.uint8, device=dev)
            y = torch.empty_like(src)
            _lib.call("sgb_relu_forward_mask_f32", src.data_ptr(), y.data_ptr(), rec.data_ptr(), n,
                      torch.cuda.current_stream().cuda_stream)
            self.t[name] = rec
        self.moments = {p: torch.zeros_like(self.t[p]) for p in self.plan["params"]}
        self.ws = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()

    def host_copy(self):
        """numpy copies of every tensor + moments (inputs for the CPU checker)."""
        out = {k: v.detach().cpu().numpy().copy() for k, v in self.t.items() if k != "grad_arena"}
        out.update({"m:" + k: v.detach().cpu().numpy().copy() for k, v in self.moments.items()})
        return out

    # -------------------------------------------------------------------- bind
    def _bind(self):
        """One (function name, argument tuple) per op; ``None`` stream slots are
        filled at run time with the current stream."""
        t, ws, L = self.t, self.ws, self.lib
        self.calls = []
        S = "STREAM"

        def p(name):
            return t[name].data_ptr()

        def geom(x, kernel, stride, pad):
            n, c, h, w = t[x].shape
            return (n, c, h, w, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1])

        for op in self.plan["ops"]:
            a, k = op.args, op.kind
            if k == "relu_bwd":
                self.calls.append(("sgb_relu_backward_f32", (p(a["dy"]), p(a["x"]), p(a["dx"]), t[a["x"]].numel(), S)))
            elif k == "relu_mask_bwd":
                self.calls.append(("sgb_relu_backward_mask_f32", (p(a["dy"]), p(a["x"]), p(a["dx"]), t[a["dx"]].numel(), S)))
            elif k == "add_relu_mask_bwd":
                self.calls.append(("sgb_add_relu_backward_mask_f32",
                                   (p(a["dy_a"]), p(a["dy_b"]), p(a["x"]), p(a["dx"]), t[a["dx"]].numel(), S)))
            elif k == "add_relu_bwd":
                self.calls.append(("sgb_add_relu_backward_f32",
                                   (p(a["dy_a"]), p(a["dy_b"]), p(a["x"]), p(a["dx"]), t[a["x"]].numel(), S)))
            elif k == "add_out":
                self.calls.append(("sgb_binary_f32", (0, p(a["a"]), p(a["b"]), p(a["out"]), t[a["out"]].numel(), S)))
            elif k in ("bn_bwd", "bn_relu_bwd", "bn_relu_mask_bwd"):
                n, c, h, w = t[a["x"]].shape
                need = L.sgb_bn_backward_workspace_bytes(n, c, h * w)
                assert need <= ws.numel()
                if k == "bn_bwd":
                    self.calls.append(("sgb_bn_backward_f32",
                                       (p(a["x"]), p(a["dy"]), p(a["scale"]), p(a["mean"]), p(a["invstd"]), p(a["dx"]),
                                        p(a["dscale"]), p(a["dbias"]), n, c, h * w, ws.data_ptr(), ws.numel(), S)))
                else:
                    self.calls.append(("sgb_bn_relu_backward_mask_f32" if k == "bn_relu_mask_bwd" else "sgb_bn_relu_backward_f32",
                                       (p(a["x"]), p(a["dy"]), p(a["relu_x"]), p(a["scale"]), p(a["mean"]),
                                        p(a["invstd"]), p(a["dx"]), p(a["dscale"]), p(a["dbias"]), n, c, h * w,
                                        ws.data_ptr(), ws.numel(), S)))
            elif k == "bn_add_relu_bwd":
                n, c, h, w = t[a["x"]].shape
                assert L.sgb_bn_backward_workspace_bytes(n, c, h * w) <= ws.numel()
                self.calls.append(("sgb_bn_add_relu_backward_f32",
                                   (p(a["x"]), p(a["dy_a"]), p(a["dy_b"]), p(a["relu_x"]), p(a["scale"]),
                                    p(a["mean"]), p(a["invstd"]), p(a["joined"]), p(a["dx"]), p(a["dscale"]),
                                    p(a["dbias"]), n, c, h * w, ws.data_ptr(), ws.numel(), S)))
            elif k == "maxpool_bwd" and self.pool_argmax:
                y_scratch = torch.empty_like(t[a["y"]])
                record = torch.empty(t[a["y"]].shape, dtype=torch.uint8, device=self.device)
                _lib.call("sgb_maxpool_forward_argmax_f32", p(a["x"]), y_scratch.data_ptr(), record.data_ptr(),
                          *geom(a["x"], a["kernel"], a["stride"], a["pad"]), torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize()
                t[a["dx"] + ".argmax"] = record
                self.calls.append(("sgb_maxpool_backward_argmax_f32",
                                   (p(a["dy"]), record.data_ptr(), p(a["dx"])) + geom(a["x"], a["kernel"], a["stride"], a["pad"]) + (S,)))
            elif k == "maxpool_bwd":
                self.calls.append(("sgb_maxpool_backward_f32",
                                   (p(a["x"]), p(a["y"]), p(a["dy"]), p(a["dx"])) + geom(a["x"], a["kernel"], a["stride"], a["pad"]) + (S,)))
            elif k == "avgpool_bwd":
                self.calls.append(("sgb_avgpool_backward_f32",
                                   (p(a["dy"]), p(a["dx"])) + geom(a["dx"], a["kernel"], a["stride"], a["pad"]) + (S,)))
            elif k == "softmax":
                r, c = t[a["x"]].shape
                self.calls.append(("sgb_softmax_rows_f32", (p(a["x"]), p(a["y"]), r, c, S)))
            elif k == "softmax_ce":
                r, c = t[a["x"]].shape
                self.calls.append(("sgb_softmax_cross_entropy_fused_f32",
                                   (p(a["x"]), p(a["t"]), r, c, float(np.float32(a["scale"])), p(a["y"]),
                                    p(a["loss"]), p(a["grad"]), S)))
            elif k == "ce_fwd":
                r, c = t[a["p"]].shape
                self.calls.append(("sgb_cross_entropy_f32", (1, r, c, p(a["p"]), p(a["t"]), p(a["loss"]), S)))
            elif k == "sum_all":
                self.calls.append(("sgb_sum_all_f32", (p(a["x"]), p(a["out"]), t[a["x"]].numel(), ws.data_ptr(), ws.numel(), S)))
            elif k == "ce_bwd":
                r, c = t[a["p"]].shape
                self.calls.append(("sgb_softmax_cross_entropy_bwd_f32", (1, r, c, p(a["p"]), p(a["t"]), p(a["grad"]), S)))
            elif k == "ce_grad":
                r, c = t[a["p"]].shape
                self.calls.append(("sgb_softmax_cross_entropy_grad_f32",
                                   (1, r, c, p(a["p"]), p(a["t"]), float(np.float32(a["scale"])), p(a["grad"]), S)))
            elif k == "scale":
                self.calls.append(("sgb_scalar_f32", (1, p(a["x"]), float(np.float32(a["c"])), p(a["x"]), t[a["x"]].numel(), S)))
            elif k == "sum_rows":
                r, c = t[a["M"]].shape
                self.calls.append(("sgb_sum_rows_f32", (p(a["M"]), p(a["v"]), r, c, ws.data_ptr(), ws.numel(), S)))
            elif k == "conv_bias_bwd":
                n, c = t[a["dy"]].shape[:2]
                hw = t[a["dy"]].numel() // (n * c)
                assert L.sgb_conv_bias_backward_workspace_bytes(n, c, hw) <= ws.numel()
                self.calls.append(("sgb_conv_bias_backward_f32",
                                   (p(a["dy"]), p(a["db"]), n, c, hw, ws.data_ptr(), ws.numel(), S)))
            elif k == "wgrad_refresh":
                # consecutive stand-ins are one run of the flat buffer
                names = ["wsyn:" + q for q in a["params"]]
                for i in range(1, len(names)):
                    assert self.wsyn_off[names[i]] == self.wsyn_off[names[i - 1]] + t[names[i - 1]].numel()
                ptrs, sizes, n = _table([t["d:" + q] for q in a["params"]])
                self._keep = getattr(self, "_keep", []) + [ptrs, sizes]
                self.calls.append(("sgb_unpack_f32", (self.wsyn_flat.data_ptr(), self.wsyn_off[names[0]], ptrs, sizes,
                                                      n, 1.0, S)))
            elif k == "fill":
                x = t[a["x"]]
                self.calls.append(("sgb_set_f32", (float(a["value"]), x.data_ptr(), x.numel(), S)))
            elif k == "grad_ready":
                self.calls.append(("grad_ready", a["param"]))
            elif k == "sync_and_update":
                self.calls.append(("sync_and_update", None))
            else:
                raise ValueError(k)
        # DistOpt policy over the gradient production order
        order = self.plan["grad_order"]
        self.grads = [t["d:" + n] for n in order]
        sizes = [g.numel() for g in self.grads]
        self.events = plan_buckets(sizes, self.threshold)
        self.flush_after = {ev[1][-1]: ev for ev in self.events}
        self.fused_tables = {ev[1][-1]: _table([self.grads[i] for i in ev[1]]) for ev in self.events if ev[0] == "fused"}
        self.single_tables = {i: _table([self.grads[i]]) for i in range(len(order))}
        names = self.plan["grad_order"]
        self.bucket_sgd = {}
        for ev in self.events:
            ps = [names[i] for i in ev[1]]
            self.bucket_sgd[ev[1][-1]] = (_table([t[n] for n in ps])[0], _table([t["d:" + n] for n in ps])[0],
                                          _table([self.moments[n] for n in ps])[0],
                                          _table([t[n] for n in ps])[1], len(ps))
        plist = self.plan["params"]
        self.sgd_tables = (_table([t[n] for n in plist])[0], _table([t["d:" + n] for n in plist])[0],
                           _table([self.moments[n] for n in plist])[0], _table([t[n] for n in plist])[1], len(plist))
        if self.dist_option.startswith("sparse") and self.comm is not None:
            self.residuals = {}
            for ev in self.events:
                tot = sum(sizes[i] for i in ev[1])
                self.residuals[ev[1][-1]] = torch.zeros(tot, device=self.device)

    # --------------------------------------------------------------------- run
    def _check(self, name, status):
        if status != 0:
            raise _lib.SgbError(name, status, self.lib.sgb_status_string(status).decode())

    def _on_grad_ready(self, idx, stream):
        """opt.py:846-862 (plain), :885-912 (half), :1030-1090 (sparse)."""
        c, L = self.comm, self.lib
        if c is None:
            return 0
        n_calls = 0
        ev = self.flush_after.get(idx)
        opt = self.dist_option
        is_direct = ev is not None and ev[0] == "direct"
        if self.profile and ev is not None:
            L.sgb_comm_profile_mark(c._h, b"bucket_ready", stream)
        if opt in ("plain", "half"):
            half = opt == "half"
            if is_direct:
                g = self.grads[idx]
                if half:
                    self._check("synch_half", L.sgb_comm_synch_half(c._h, g.data_ptr(), g.numel(), stream))
                else:
                    self._check("synch", L.sgb_comm_synch(c._h, g.data_ptr(), g.numel(), 0, stream))
                self._sgd_bucket(idx)
                return 1
            ptrs, sizes, n = self.single_tables[idx]
            if half:
                self._check("stage_half", L.sgb_comm_fused_synch_half(c._h, ptrs, sizes, n, 0, stream))
            else:
                self._check("stage", L.sgb_comm_fused_synch(c._h, ptrs, sizes, n, 0, 0, stream))
            n_calls += 1
            if ev is not None:
                ptrs, sizes, n = self.fused_tables[idx]
                if half:
                    self._check("flush_half", L.sgb_comm_fused_synch_half(c._h, ptrs, sizes, n, 1, stream))
                else:
                    self._check("flush", L.sgb_comm_fused_synch(c._h, ptrs, sizes, n, 0, 1, stream))
                self._sgd_bucket(idx)
                n_calls += 2
            return n_calls
        # sparse options: nothing is staged, the whole bucket is handed over at flush time
        if ev is None:
            return 0
        topk = opt == "sparseTopK"
        ptrs, sizes, n = self.single_tables[idx] if is_direct else self.fused_tables[idx]
        self._check("sparsification", L.sgb_comm_sparsification(
            c._h, ptrs, sizes, n, self.residuals[idx].data_ptr(), float(self.spars), int(topk), stream))
        return 1

    def _sgd_bucket(self, idx):
        """The bucket's parameters are updated on the side stream on which its
        reduced gradients land (never on the NCCL stream: the next bucket's
        all-reduce does not wait for this update)."""
        if not self.update_on_arrival:
            return
        L, h = self.lib, self.comm._h
        side = L.sgb_comm_result_stream(h)
        which = [L.sgb_comm_stream(h, w) for w in (0, 1, 2)].index(side)
        pp, gp, mp, sizes, n = self.bucket_sgd[idx]
        scale = float(np.float32(1.0) / np.float32(self.world))
        L.sgb_comm_profile_range(h, b"sgd_update_bucket", which, 1)
        self._check("sgd", L.sgb_sgd_update_multi_f32(pp, gp, mp, sizes, n, self.lr, self.momentum, 0.0,
                                                       self.weight_decay, 0, scale, side))
        L.sgb_comm_profile_range(h, b"sgd_update_bucket", which, 0)

    def run_step(self):
        """Enqueues one full step on the current stream (+ the communicator's
        side streams).  Returns the number of C-ABI calls issued."""
        L = self.lib
        stream = torch.cuda.current_stream().cuda_stream
        order_index = {n: i for i, n in enumerate(self.plan["grad_order"])}
        ncalls = 0
        for name, args in self.calls:
            if name == "grad_ready":
                ncalls += self._on_grad_ready(order_index[args], stream)
            elif name == "sync_and_update":
                if self.comm is not None:
                    self._check("wait", L.sgb_comm_wait(self.comm._h, stream))
                if self.update_on_arrival:
                    continue                  # every bucket was updated as it arrived
                pp, gp, mp, sizes, n = self.sgd_tables
                scale = float(np.float32(1.0) / np.float32(self.world))
                self._check("sgd", L.sgb_sgd_update_multi_f32(pp, gp, mp, sizes, n, self.lr, self.momentum, 0.0,
                                                               self.weight_decay, 0, scale, stream))
                ncalls += 1
            else:
                st = getattr(L, name)(*[stream if a == "STREAM" else a for a in args])
                if st != 0:
                    self._check(name, st)
                ncalls += 1
        return ncalls

    def capture(self):
        """Captures one step into a CUDA graph (after a warm-up step has run)."""
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                self.run_step()
        torch.cuda.current_stream().wait_stream(s)
        self.graph = g
        return g

    def release_graph(self):
        """Drops the captured step.  Must be called before the communicator is
        closed: NCCL keeps a communicator alive (its destroy call waits) for as
        long as a CUDA graph that captured its collectives exists."""
        self.graph = None

    def loss(self):
        return self.t["loss"]
