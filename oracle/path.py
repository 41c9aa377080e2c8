"""CPU executor of a hot-path plan (``singa_b200.resnet50_path.build_plan``)
on numpy arrays, using the oracle's C restatement op by op.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``): the end-to-end parity
check of the GPU executor, the smoke check and the timed CPU baseline of the
benchmark walk the same op list through this class.
"""
import numpy as np

from . import comm, cpu


class OraclePath(object):
    def __init__(self, plan, tensors, lr=0.1, momentum=0.9, weight_decay=1e-5, world=1,
                 dist_option="plain"):
        """``tensors``: dict name -> numpy array (e.g. HotPathGPU.host_copy());
        moments under "m:<param>".  Arrays are updated in place."""
        self.plan, self.t = plan, tensors
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.world, self.dist_option = world, dist_option

    def run_step(self):
        t = self.t
        for op in self.plan["ops"]:
            a, k = op.args, op.kind
            if k == "relu_bwd":
                t[a["dx"]][...] = cpu.relu_backward(t[a["dy"]], t[a["x"]])
            elif k == "relu_mask_bwd":        # the bit record encodes x > 0: recompute it from the input
                t[a["dx"]][...] = cpu.relu_backward(t[a["dy"]], t[a["x_ref"]])
            elif k == "add_relu_bwd":
                t[a["dx"]][...] = cpu.relu_backward(t[a["dy_a"]] + t[a["dy_b"]], t[a["x"]])
            elif k == "add_relu_mask_bwd":
                t[a["dx"]][...] = cpu.relu_backward(t[a["dy_a"]] + t[a["dy_b"]], t[a["x_ref"]])
            elif k == "add_out":
                t[a["out"]][...] = t[a["a"]] + t[a["b"]]
            elif k in ("bn_bwd", "bn_relu_bwd", "bn_relu_mask_bwd", "bn_add_relu_bwd"):
                if k == "bn_add_relu_bwd":
                    t[a["joined"]][...] = cpu.relu_backward(t[a["dy_a"]] + t[a["dy_b"]], t[a["relu_x"]])
                    dy = t[a["joined"]]
                else:
                    dy = t[a["dy"]]
                if k == "bn_relu_bwd":
                    dy = cpu.relu_backward(dy, t[a["relu_x"]])
                if k == "bn_relu_mask_bwd":
                    dy = cpu.relu_backward(dy, t[a["x_ref"]])
                dx, ds, db = cpu.bn_backward(dy, t[a["x"]], t[a["scale"]], t[a["mean"]], t[a["invstd"]])
                t[a["dx"]][...] = dx
                t[a["dscale"]][...] = ds
                t[a["dbias"]][...] = db
            elif k == "maxpool_bwd":
                t[a["dx"]][...] = cpu.maxpool_backward(t[a["dy"]], t[a["x"]], a["kernel"], a["stride"], a["pad"])
            elif k == "avgpool_bwd":
                t[a["dx"]][...] = cpu.avgpool_backward(t[a["dy"]], t[a["dx"]].shape, a["kernel"], a["stride"], a["pad"])
            elif k == "softmax":
                t[a["y"]][...] = cpu.softmax(t[a["x"]])
            elif k == "softmax_ce":
                t[a["y"]][...] = cpu.softmax(t[a["x"]])
                t[a["loss"]][...] = cpu.cross_entropy_fwd(t[a["y"]], t[a["t"]])
                t[a["grad"]][...] = cpu.softmax_cross_entropy_bwd(t[a["y"]], t[a["t"]]) * np.float32(a["scale"])
            elif k == "ce_fwd":
                t[a["loss"]][...] = cpu.cross_entropy_fwd(t[a["p"]], t[a["t"]])
            elif k == "sum_all":
                t[a["out"]][0] = cpu.sum_all(t[a["x"]])
            elif k == "ce_bwd":
                t[a["grad"]][...] = cpu.softmax_cross_entropy_bwd(t[a["p"]], t[a["t"]])
            elif k == "ce_grad":
                t[a["grad"]][...] = cpu.softmax_cross_entropy_bwd(t[a["p"]], t[a["t"]]) * np.float32(a["scale"])
            elif k == "scale":
                cpu.scale_inplace(t[a["x"]], np.float32(a["c"]))
            elif k == "sum_rows":
                t[a["v"]][...] = cpu.sum_rows(t[a["M"]])
            elif k == "conv_bias_bwd":
                t[a["db"]][...] = cpu.conv_bias_backward(t[a["dy"]])
            elif k == "wgrad_refresh":
                for p in a["params"]:
                    t["d:" + p][...] = t["wsyn:" + p]
            elif k == "fill":       # every parameter gradient := value (the GPU fills its gradient arena)
                for p in self.plan["params"]:
                    t["d:" + p][...] = np.float32(a["value"])
            elif k == "grad_ready":
                pass     # one rank: the all-reduce of a single contribution is the identity
            elif k == "sync_and_update":
                self._update()
            else:
                raise ValueError(k)

    def _update(self):
        t = self.t
        scale = np.float32(1.0) / np.float32(self.world)
        for p in self.plan["params"]:
            g = t["d:" + p]
            if self.dist_option == "half":
                g = comm.allreduce_half([g])
            if self.world != 1:
                g = (g * scale).astype(np.float32)
            g = np.ascontiguousarray(g, np.float32).copy()
            cpu.sgd_update(t[p], g, t["m:" + p], self.lr, momentum=self.momentum,
                           weight_decay=self.weight_decay)


def make_tensors(plan, seed=0):
    """Seeded numpy tensors for a plan (same roles and value distributions as
    the GPU executor's, generated on the host)."""
    rng = np.random.default_rng(seed)
    T = plan["tensors"]
    t = {}
    for name, spec in T.items():
        k = spec.kind
        if k == "label":
            t[name] = rng.integers(0, T["logits"].shape[1], spec.shape).astype(np.int32)
        elif k == "act":
            bn_in = name.endswith(".x") and (".bn" in name or name == "bn1.x")
            t[name] = rng.standard_normal(spec.shape, dtype=np.float32)
            if bn_in:
                t[name] = t[name] * np.float32(1.5) + np.float32(0.2)
        elif k == "syn":
            t[name] = rng.standard_normal(spec.shape, dtype=np.float32) * np.float32(1e-2)
        elif k == "param":
            if name.endswith(".scale"):
                t[name] = np.ones(spec.shape, np.float32)
            elif name.endswith(".bias") or name == "fc.b":
                t[name] = np.zeros(spec.shape, np.float32)
            else:
                t[name] = rng.standard_normal(spec.shape, dtype=np.float32) * np.float32(0.05)
        elif k in ("pgrad", "wsyn"):
            t[name] = rng.standard_normal(spec.shape, dtype=np.float32) * np.float32(1e-3)
        elif k == "mask":
            continue                              # the CPU checker recomputes the decisions from the input
        else:
            t[name] = np.zeros(spec.shape, np.float32)
    for name in list(T):
        if name.endswith(".mean"):
            base = name[:-5]
            mean, invstd = cpu.bn_stats(t[base + ".x"])
            t[base + ".mean"], t[base + ".invstd"] = mean, invstd
    for p in plan["params"]:
        t["m:" + p] = np.zeros(T[p].shape, np.float32)
    return t
