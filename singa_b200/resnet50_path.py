"""The ResNet-50 backward + gradient-sync + update hot path as a list of ops.

This is the workload of the headline benchmark: the sequence of backward
calls that the reference's Python autograd issues for its ResNet-50
(examples/cnn/model/resnet.py: Bottleneck blocks [3, 4, 6, 3], 7x7 stem,
3x3/2 max pool, 7x7 average pool, 1000-way linear) at batch 32/GPU, 224x224
input, followed by DistOpt's bucketed gradient synchronisation and the SGD
update of the 161 parameter tensors.

The Conv/Linear contractions are NOT part of this path (they stay on
cuDNN/cuBLAS in the reference), so the gradients they would produce are
stand-in tensors with fixed seeded content: the activation gradient a
conv-backward-data call would write, and the weight gradient a
conv-backward-filter call would write.  Everything else - ReLU backward,
batch-norm backward, the residual joins, max/avg-pool backward,
softmax-cross-entropy forward/backward, the bias-gradient reduction, the
gradient synchronisation and the optimizer - is computed.

``build_plan`` is pure python (no device): it returns tensor specs and an op
list that an executor (GPU: ``HotPathGPU`` below; CPU checker: the oracle
executor in bench.py/tests) walks in order.
"""
from collections import namedtuple

Tensor = namedtuple("Tensor", "name shape kind")
# kind: "act"   stored forward activation (seeded content)
#       "stat"  per-channel BN statistic / scale
#       "syn"   stand-in for a contraction's output gradient (seeded content)
#       "grad"  activation gradient produced on the path (scratch)
#       "param" parameter, "pgrad" parameter gradient, "label", "misc"

Op = namedtuple("Op", "kind args")


def conv_out(h, k, stride, pad):
    return (h + 2 * pad - k) // stride + 1


def build_plan(batch=32, image=224, num_classes=1000, fused=False, blocks=(3, 4, 6, 3), join_bn=False):
    """Returns dict(tensors, ops, params, grad_order, stats).

    fused=False: one op per reference call (ReLUBackward, GpuBatchNormBackward,
    ``+=`` join, ...).  fused=True: the join is folded into the following
    ReLUBackward and ReLUBackward into the following GpuBatchNormBackward
    (same results, fewer passes over memory).  join_bn=True (with fused) also
    folds the join + ReLUBackward at a block's end into the batch-norm
    backward after it; see fuse_plan for why that is not the default."""
    T, ops, params = {}, [], []
    B = batch

    def tensor(name, shape, kind):
        assert name not in T, name
        T[name] = Tensor(name, tuple(shape), kind)
        return name

    def param(name, shape):
        tensor(name, shape, "param")
        tensor("d:" + name, shape, "pgrad")
        params.append(name)
        return name

    def bn(name, c, h):
        param(name + ".scale", (c,))
        param(name + ".bias", (c,))
        tensor(name + ".x", (B, c, h, h), "act")          # conv output = BN input
        tensor(name + ".mean", (c,), "stat")
        tensor(name + ".invstd", (c,), "stat")

    # ---------------------------------------------------------------- forward walk
    fwd = []          # structural records used to emit the backward ops
    h = conv_out(image, 7, 2, 3)
    param("conv1.W", (64, 3, 7, 7))
    bn("bn1", 64, h)
    tensor("relu.x", (B, 64, h, h), "act")                 # BN output = ReLU input
    hp = conv_out(h, 3, 2, 1)
    tensor("maxpool.x", (B, 64, h, h), "act")              # ReLU output
    tensor("maxpool.y", (B, 64, hp, hp), "act")
    stem = dict(h=h, hp=hp)
    inpl, h = 64, hp
    for li, (planes, nblk, stride) in enumerate(zip((64, 128, 256, 512), blocks, (1, 2, 2, 2)), 1):
        for b in range(nblk):
            s = stride if b == 0 else 1
            n = "layer%d.%d" % (li, b)
            hin = h
            h1 = conv_out(hin, 1, 1, 0)
            param(n + ".conv1.W", (planes, inpl, 1, 1)); bn(n + ".bn1", planes, h1)
            tensor(n + ".relu1.x", (B, planes, h1, h1), "act")
            h2 = conv_out(h1, 3, s, 1)
            param(n + ".conv2.W", (planes, planes, 3, 3)); bn(n + ".bn2", planes, h2)
            tensor(n + ".relu2.x", (B, planes, h2, h2), "act")
            h3 = conv_out(h2, 1, 1, 0)
            param(n + ".conv3.W", (planes * 4, planes, 1, 1)); bn(n + ".bn3", planes * 4, h3)
            down = b == 0
            if down:
                param(n + ".down.conv.W", (planes * 4, inpl, 1, 1)); bn(n + ".down.bn", planes * 4, h3)
            tensor(n + ".relu3.x", (B, planes * 4, h3, h3), "act")   # add output
            fwd.append(dict(name=n, cin=inpl, planes=planes, hin=hin, h1=h1, h2=h2, h3=h3, down=down))
            inpl, h = planes * 4, h3
    param("fc.W", (inpl, num_classes))
    param("fc.b", (num_classes,))
    tensor("labels", (B,), "label")
    tensor("logits", (B, num_classes), "act")
    tensor("prob", (B, num_classes), "grad")
    tensor("loss_vec", (B,), "grad")
    tensor("loss", (1,), "grad")
    tensor("dlogits", (B, num_classes), "grad")
    tensor("avgpool.dy", (B, inpl, 1, 1), "syn")           # from the fc Matmul backward (cuBLAS)
    tensor("d:fc.W.syn", (1,), "misc")

    # ---------------------------------------------------------------- backward ops
    grad_order = []

    def ready(pname):
        grad_order.append(pname)
        ops.append(Op("grad_ready", dict(param=pname)))

    def syn(name, shape):
        return tensor(name, shape, "syn")

    def scratch(name, shape):
        return tensor(name, shape, "grad")

    # head: loss forward, softmax-CE backward (+1/N), bias gradient, avg-pool backward
    if fused:
        ops.append(Op("softmax_ce", dict(x="logits", t="labels", y="prob", loss="loss_vec", grad="dlogits",
                                         scale=1.0 / B)))
        ops.append(Op("sum_all", dict(x="loss_vec", out="loss")))
    else:
        ops.append(Op("softmax", dict(x="logits", y="prob")))
        ops.append(Op("ce_fwd", dict(p="prob", t="labels", loss="loss_vec")))
        ops.append(Op("sum_all", dict(x="loss_vec", out="loss")))
    if not fused:
        ops.append(Op("ce_bwd", dict(p="prob", t="labels", grad="dlogits")))
        ops.append(Op("scale", dict(x="dlogits", c=1.0 / B)))
    ops.append(Op("sum_rows", dict(M="dlogits", v="d:fc.b")))
    ready("fc.b")
    ready("fc.W")                                          # cuBLAS weight gradient: stand-in content
    hlast = fwd[-1]["h3"]
    dcur = scratch("avgpool.dx", (B, inpl, hlast, hlast))
    ops.append(Op("avgpool_bwd", dict(dy="avgpool.dy", dx=dcur, kernel=(hlast, hlast), stride=(1, 1), pad=(0, 0))))

    # dcur = gradient w.r.t. the output of the current block (after relu3)
    pending_join = None    # (a, b): gradient is a + b, not yet materialised (fused mode)
    for blk in reversed(fwd):
        n, p4, pl = blk["name"], blk["planes"] * 4, blk["planes"]
        shape3 = (B, p4, blk["h3"], blk["h3"])
        d_add = scratch(n + ".d_add", shape3)
        join = None
        if pending_join is not None and not join_bn:
            ops.append(Op("add_relu_bwd", dict(dy_a=pending_join[0], dy_b=pending_join[1], x=n + ".relu3.x", dx=d_add)))
            pending_join = None
        elif pending_join is not None:
            # folded into the batch-norm backward that follows (bn3 reads d_add first)
            join = dict(dy_a=pending_join[0], dy_b=pending_join[1], relu_x=n + ".relu3.x", joined=d_add)
            pending_join = None
        else:
            ops.append(Op("relu_bwd", dict(dy=dcur, x=n + ".relu3.x", dx=d_add)))

        def bn_bwd(bnname, dy, relu_x=None, join=None):
            c, hh = T[bnname + ".x"].shape[1], T[bnname + ".x"].shape[2]
            dx = scratch(bnname + ".dx", (B, c, hh, hh))
            args = dict(dy=dy, x=bnname + ".x", scale=bnname + ".scale", mean=bnname + ".mean",
                        invstd=bnname + ".invstd", dx=dx, dscale="d:" + bnname + ".scale",
                        dbias="d:" + bnname + ".bias")
            if join is not None:
                del args["dy"]
                ops.append(Op("bn_add_relu_bwd", dict(args, **join)))
            elif relu_x is not None and fused:
                ops.append(Op("bn_relu_bwd", dict(args, relu_x=relu_x)))
            else:
                if relu_x is not None:
                    masked = scratch(bnname + ".dy_masked", (B, c, hh, hh))
                    ops.append(Op("relu_bwd", dict(dy=dy, x=relu_x, dx=masked)))
                    args["dy"] = masked
                ops.append(Op("bn_bwd", args))
            ready(bnname + ".bias")
            ready(bnname + ".scale")
            return dx

        # main branch: bn3 <- conv3 <- relu2 <- bn2 <- conv2 <- relu1 <- bn1 <- conv1
        bn_bwd(n + ".bn3", d_add, join=join)
        ready(n + ".conv3.W")
        g2 = syn(n + ".conv3.dgrad", (B, pl, blk["h2"], blk["h2"]))      # cudnn bwd-data output
        bn_bwd(n + ".bn2", g2, relu_x=n + ".relu2.x")
        ready(n + ".conv2.W")
        g1 = syn(n + ".conv2.dgrad", (B, pl, blk["h1"], blk["h1"]))
        bn_bwd(n + ".bn1", g1, relu_x=n + ".relu1.x")
        ready(n + ".conv1.W")
        dx_main = syn(n + ".conv1.dgrad", (B, blk["cin"], blk["hin"], blk["hin"]))
        if blk["down"]:
            bn_bwd(n + ".down.bn", d_add)
            ready(n + ".down.conv.W")
            dx_res = syn(n + ".down.dgrad", (B, blk["cin"], blk["hin"], blk["hin"]))
        else:
            dx_res = d_add                                 # identity shortcut
        # join of the two gradients reaching the block input: dxs_[y_idx] += dx
        if fused and blk is not fwd[0]:
            pending_join = (dx_main, dx_res)
            dcur = None
        else:
            joined = scratch(n + ".d_in", (B, blk["cin"], blk["hin"], blk["hin"]))
            ops.append(Op("add_out", dict(a=dx_main, b=dx_res, out=joined)))
            dcur = joined

    # stem: maxpool <- relu <- bn1 <- conv1
    d_pool = scratch("maxpool.dx", T["maxpool.x"].shape)
    ops.append(Op("maxpool_bwd", dict(x="maxpool.x", y="maxpool.y", dy=dcur, dx=d_pool,
                                      kernel=(3, 3), stride=(2, 2), pad=(1, 1))))
    c, hh = 64, stem["h"]
    dx = scratch("bn1.dx", (B, c, hh, hh))
    bnargs = dict(dy=d_pool, x="bn1.x", scale="bn1.scale", mean="bn1.mean", invstd="bn1.invstd",
                  dx=dx, dscale="d:bn1.scale", dbias="d:bn1.bias")
    if fused:
        ops.append(Op("bn_relu_bwd", dict(bnargs, relu_x="relu.x")))
    else:
        masked = scratch("bn1.dy_masked", (B, c, hh, hh))
        ops.append(Op("relu_bwd", dict(dy=d_pool, x="relu.x", dx=masked)))
        ops.append(Op("bn_bwd", dict(bnargs, dy=masked)))
    ready("bn1.bias")
    ready("bn1.scale")
    ready("conv1.W")
    ops.append(Op("sync_and_update", dict()))
    del T["d:fc.W.syn"]
    return dict(tensors=T, ops=ops, params=params, grad_order=grad_order, batch=B)


READS = {
    "relu_bwd": ("dy", "x"), "add_relu_bwd": ("dy_a", "dy_b", "x"), "add_out": ("a", "b"),
    "relu_mask_bwd": ("dy", "x"), "add_relu_mask_bwd": ("dy_a", "dy_b", "x"),
    "bn_relu_mask_bwd": ("dy", "relu_x", "x", "scale", "mean", "invstd"),
    "bn_bwd": ("dy", "x", "scale", "mean", "invstd"),
    "bn_relu_bwd": ("dy", "relu_x", "x", "scale", "mean", "invstd"),
    "bn_add_relu_bwd": ("dy_a", "dy_b", "relu_x", "x", "scale", "mean", "invstd"),
    "maxpool_bwd": ("x", "y", "dy"), "avgpool_bwd": ("dy",), "softmax": ("x",), "ce_fwd": ("p", "t"),
    "sum_all": ("x",), "ce_bwd": ("p", "t"), "ce_grad": ("p", "t"), "scale": ("x",), "sum_rows": ("M",),
    "conv_bias_bwd": ("dy",), "softmax_ce": ("x", "t"),
}


def fuse_plan(plan, join_bn=False):
    """Peephole fusion over a recorded op list (the counterpart of a pass over
    the reference's buffered Graph nodes, keyed on the op kinds):

      add_out(a, b -> t) ; relu_bwd(dy=t, x -> dx)       =>  add_relu_bwd(a, b, x -> dx)
      relu_bwd(dy, x=r -> m) ; bn_bwd(dy=m, ...)         =>  bn_relu_bwd(dy, relu_x=r, ...)
      add_relu_bwd(a, b, x=r -> t) ; bn_bwd(dy=t, ...)   =>  bn_add_relu_bwd(a, b, relu_x=r, joined=t, ...)
                                                             (only with join_bn=True)
      ce_bwd(p, t -> g) ; scale(g, c)                    =>  ce_grad(p, t, c -> g)
      softmax(x -> p) ; ce_fwd(p, t -> l) ; ... ; ce_grad(p, t, c -> g)
                                                         =>  softmax_ce(x, t, c -> p, l, g)   (at softmax's place)

    A pair is fused only when the intermediate tensor has no other reader;
    the intermediate then disappears from the plan.  The last rule is the
    exception: the joined gradient `t` stays (the shortcut branch reads it
    later) and is written by the fused op, which must be its FIRST reader.
    It is off by default because it does not pay on B200: it saves 4 of 28
    bytes per element but moves the join's 16 bytes from a streaming kernel
    that runs at the copy bandwidth into the batch-norm kernel that reaches
    about 0.7 of it (measured 130 us fused against 58 + 67 us at 32x256x56x56).
    Results are unchanged bit for bit (the fused kernels perform the same
    roundings)."""
    ops = list(plan["ops"])
    readers = {}
    for i, op in enumerate(ops):
        for key in READS.get(op.kind, ()):
            readers.setdefault(op.args[key], []).append(i)
    dead, out, T = set(), [], dict(plan["tensors"])
    producer = {}
    for i, op in enumerate(ops):
        k, a = op.kind, op.args
        if k == "relu_bwd" and a["dy"] in producer and out[producer[a["dy"]]].kind == "add_out" \
                and producer[a["dy"]] not in dead and readers.get(a["dy"]) == [i]:
            j = producer[a["dy"]]
            src = out[j].args
            dead.add(j)
            T.pop(a["dy"], None)
            op = Op("add_relu_bwd", dict(dy_a=src["a"], dy_b=src["b"], x=a["x"], dx=a["dx"]))
        elif k == "bn_bwd" and a["dy"] in producer and out[producer[a["dy"]]].kind == "relu_bwd" \
                and producer[a["dy"]] not in dead and readers.get(a["dy"]) == [i]:
            # keyed on the op as already rewritten: a relu_bwd that absorbed a join is an
            # add_relu_bwd by now and is left alone here (join_bn handles that pair)
            j = producer[a["dy"]]
            src = out[j].args
            dead.add(j)
            T.pop(a["dy"], None)
            op = Op("bn_relu_bwd", dict(a, dy=src["dy"], relu_x=src["x"]))
        elif join_bn and k == "bn_bwd" and a["dy"] in producer and out[producer[a["dy"]]].kind == "add_relu_bwd" \
                and producer[a["dy"]] not in dead and readers.get(a["dy"], [None])[0] == i:
            j = producer[a["dy"]]
            src = out[j].args
            dead.add(j)
            rest = {key: v for key, v in a.items() if key != "dy"}
            op = Op("bn_add_relu_bwd", dict(rest, dy_a=src["dy_a"], dy_b=src["dy_b"], relu_x=src["x"],
                                            joined=a["dy"]))
        elif k == "scale" and a["x"] in producer and out[producer[a["x"]]].kind == "ce_bwd" \
                and producer[a["x"]] not in dead:
            j = producer[a["x"]]
            src = out[j].args
            dead.add(j)
            op = Op("ce_grad", dict(p=src["p"], t=src["t"], scale=a["c"], grad=a["x"]))
        out.append(op)
        for key in ("dx", "out", "grad", "y", "loss", "v", "joined"):
            if key in op.args and isinstance(op.args[key], str):
                producer[op.args[key]] = i
    # a fused relu_bwd may itself have consumed an add_out: drop everything marked dead
    fused_ops = [op for i, op in enumerate(out) if i not in dead]
    fused_ops = _fuse_loss_head(fused_ops)
    return dict(plan, ops=fused_ops, tensors=T)


def _fuse_loss_head(ops):
    """softmax ; ce_fwd ; (ops that touch neither p nor the gradient) ; ce_grad on
    the same probabilities and integer targets -> one softmax_ce op where the
    softmax stood.  The probabilities stay an output (later readers keep working)."""
    ops = list(ops)
    for i, op in enumerate(ops):
        if op.kind != "softmax":
            continue
        pname = op.args["y"]
        fwd = next((j for j in range(i + 1, len(ops)) if ops[j].kind == "ce_fwd" and ops[j].args["p"] == pname), None)
        grd = next((j for j in range(i + 1, len(ops)) if ops[j].kind == "ce_grad" and ops[j].args["p"] == pname), None)
        if fwd is None or grd is None or fwd > grd or ops[fwd].args["t"] != ops[grd].args["t"]:
            continue
        gname, lname = ops[grd].args["grad"], ops[fwd].args["loss"]
        between = [ops[j] for j in range(i + 1, grd) if j != fwd]
        touched = set()
        for o in between:
            touched.update(v for v in o.args.values() if isinstance(v, str))
        if gname in touched or pname in touched:
            continue
        fused = Op("softmax_ce", dict(x=op.args["x"], t=ops[fwd].args["t"], y=pname, loss=lname, grad=gname,
                                      scale=ops[grd].args["scale"]))
        return ops[:i] + [fused] + [o for j, o in enumerate(ops[i + 1:], i + 1) if j not in (fwd, grd)]
    return ops


WRITES = {
    "relu_bwd": ("dx",), "add_relu_bwd": ("dx",), "add_out": ("out",),
    "relu_mask_bwd": ("dx",), "add_relu_mask_bwd": ("dx",), "bn_relu_mask_bwd": ("dx", "dscale", "dbias"),
    "bn_bwd": ("dx", "dscale", "dbias"), "bn_relu_bwd": ("dx", "dscale", "dbias"),
    "bn_add_relu_bwd": ("joined", "dx", "dscale", "dbias"), "maxpool_bwd": ("dx",), "avgpool_bwd": ("dx",),
    "softmax": ("y",), "ce_fwd": ("loss",), "sum_all": ("out",), "ce_bwd": ("grad",), "ce_grad": ("grad",),
    "scale": ("x",), "sum_rows": ("v",), "conv_bias_bwd": ("db",), "softmax_ce": ("y", "loss", "grad"),
}


def add_wgrad_refresh(plan, where="start"):
    """Rewrites, every step, the parameter gradients that no op of the path
    produces (the weight gradients of the Conv/Linear contractions) from
    pristine stand-in copies "wsyn:<param>".  This stands for the write the
    contraction's backward-filter call performs in the reference; without it a
    stand-in gradient that is all-reduced in place would be multiplied by the
    world size on every step.  where="start": one multi-tensor copy at the
    beginning of the step; where="each": one copy right before each such
    gradient is reported ready (the position of the contraction)."""
    written = set()
    for op in plan["ops"]:
        for key in WRITES.get(op.kind, ()):
            written.add(op.args[key])
    stand = [p for p in plan["grad_order"] if "d:" + p not in written]
    T = dict(plan["tensors"])
    for p in stand:
        T["wsyn:" + p] = Tensor("wsyn:" + p, T["d:" + p].shape, "wsyn")
    if where == "start":
        ops = [Op("wgrad_refresh", dict(params=tuple(stand)))] + list(plan["ops"])
    else:
        ops, todo = [], set(stand)
        for op in plan["ops"]:
            if op.kind == "grad_ready" and op.args["param"] in todo:
                ops.append(Op("wgrad_refresh", dict(params=(op.args["param"],))))
            ops.append(op)
    return dict(plan, ops=ops, tensors=T)


def mask_plan(plan):
    """Rewrites every ReLU backward (alone, joined, or folded into a batch-norm
    backward) to consume the forward partner's one-bit-per-element record
    "mask:<relu input>" instead of the stored ReLU input.  Opt-in: it changes
    what the backward pass consumes.  The ops keep the name of the original
    input under "x_ref" so that a checker can recompute the decisions."""
    T = dict(plan["tensors"])
    rename = {"relu_bwd": ("relu_mask_bwd", "x"), "add_relu_bwd": ("add_relu_mask_bwd", "x"),
              "bn_relu_bwd": ("bn_relu_mask_bwd", "relu_x")}
    ops = []
    for op in plan["ops"]:
        if op.kind in rename:
            kind, key = rename[op.kind]
            src = op.args[key]
            mname = "mask:" + src
            if mname not in T:
                T[mname] = Tensor(mname, T[src].shape, "mask")
            args = dict(op.args)
            args[key] = mname
            args["x_ref"] = src
            op = Op(kind, args)
        ops.append(op)
    return dict(plan, ops=ops, tensors=T)


def numel(shape):
    n = 1
    for s in shape:
        n *= s
    return n


def algorithmic_bytes(plan, world=1, pool_argmax=False):
    """Bytes each op must move at minimum (fp32), by op family - the figures the
    roofline fraction is computed on.  BN backward counts 12 B/element (read x,
    read dy, write dx) + 20 B/channel whatever the implementation moves; the
    fused forms add 4 B/element for the ReLU mask / second addend."""
    T = plan["tensors"]
    out = {}

    def add(k, v):
        out[k] = out.get(k, 0) + v

    for op in plan["ops"]:
        a = op.args
        if op.kind == "relu_bwd":
            add("relu_bwd", 12 * numel(T[a["x"]].shape))
        elif op.kind == "add_relu_bwd":
            add("add_relu_bwd", 16 * numel(T[a["x"]].shape))
        elif op.kind == "relu_mask_bwd":                 # dy, dx and one bit per element
            add("relu_mask_bwd", 8 * numel(T[a["dx"]].shape) + numel(T[a["dx"]].shape) // 8)
        elif op.kind == "add_relu_mask_bwd":
            add("add_relu_mask_bwd", 12 * numel(T[a["dx"]].shape) + numel(T[a["dx"]].shape) // 8)
        elif op.kind == "bn_relu_mask_bwd":
            s = T[a["x"]].shape
            add("bn_relu_mask_bwd", 12 * numel(s) + numel(s) // 8 + 20 * s[1])
        elif op.kind == "add_out":
            add("join", 12 * numel(T[a["out"]].shape))
        elif op.kind == "bn_bwd":
            s = T[a["x"]].shape
            add("bn_bwd", 12 * numel(s) + 20 * s[1])
        elif op.kind == "bn_relu_bwd":
            s = T[a["x"]].shape
            add("bn_relu_bwd", 16 * numel(s) + 20 * s[1])
        elif op.kind == "bn_add_relu_bwd":
            s = T[a["x"]].shape                   # reads x, dy_a, dy_b, relu_x; writes joined, dx
            add("bn_add_relu_bwd", 24 * numel(s) + 20 * s[1])
        elif op.kind == "maxpool_bwd" and pool_argmax:   # dy, one record byte per window, dx
            add("maxpool_bwd", 4 * (numel(T[a["x"]].shape) + numel(T[a["y"]].shape)) + numel(T[a["y"]].shape))
        elif op.kind == "maxpool_bwd":
            add("maxpool_bwd", 4 * (2 * numel(T[a["x"]].shape) + 2 * numel(T[a["y"]].shape)))
        elif op.kind == "avgpool_bwd":
            add("avgpool_bwd", 4 * (numel(T[a["dy"]].shape) + numel(T[a["dx"]].shape)))
        elif op.kind in ("ce_bwd", "ce_grad"):
            add("softmax_ce", 8 * numel(T[a["p"]].shape))
        elif op.kind == "softmax":
            add("softmax_ce", 8 * numel(T[a["x"]].shape))
        elif op.kind == "softmax_ce":
            add("softmax_ce", 12 * numel(T[a["x"]].shape))       # read logits, write prob and grad
        elif op.kind == "scale":
            add("softmax_ce", 8 * numel(T[a["x"]].shape))
        elif op.kind == "sum_rows":
            add("bias_grad", 4 * numel(T[a["M"]].shape))
        elif op.kind == "wgrad_refresh":                         # read the stand-in, write the gradient
            add("wgrad_standin", 8 * sum(numel(T["d:" + p].shape) for p in a["params"]))
    nparam = sum(numel(T[p].shape) for p in plan["params"])
    add("sgd", 20 * nparam)
    return out, nparam


# ---------------------------------------------------------------- small configs
def build_mlp_plan(batch=256, dims=(784, 4096, 4096, 10)):
    """Backward + update path of the reference MLP (Linear-ReLU-Linear-ReLU-Linear,
    softmax cross entropy; examples/mlp/model.py shape family; benchmark configuration 1).
    Matmul gradients are stand-ins (cuBLAS); the bias gradients (SumRows), ReLU
    backward, softmax-CE and the SGD update are computed."""
    T, ops, params, order = {}, [], [], []
    B = batch

    def tensor(name, shape, kind):
        T[name] = Tensor(name, tuple(shape), kind)
        return name

    def param(name, shape):
        tensor(name, shape, "param")
        tensor("d:" + name, shape, "pgrad")
        params.append(name)

    nl = len(dims) - 1
    for i in range(nl):
        param("fc%d.W" % i, (dims[i], dims[i + 1]))
        param("fc%d.b" % i, (dims[i + 1],))
        if i < nl - 1:
            tensor("relu%d.x" % i, (B, dims[i + 1]), "act")
    tensor("labels", (B,), "label")
    tensor("logits", (B, dims[-1]), "act")
    for n, shp in (("prob", (B, dims[-1])), ("loss_vec", (B,)), ("loss", (1,)), ("dlogits", (B, dims[-1]))):
        tensor(n, shp, "grad")

    def ready(p):
        order.append(p)
        ops.append(Op("grad_ready", dict(param=p)))

    ops.append(Op("softmax", dict(x="logits", y="prob")))
    ops.append(Op("ce_fwd", dict(p="prob", t="labels", loss="loss_vec")))
    ops.append(Op("sum_all", dict(x="loss_vec", out="loss")))
    ops.append(Op("ce_bwd", dict(p="prob", t="labels", grad="dlogits")))
    ops.append(Op("scale", dict(x="dlogits", c=1.0 / B)))
    dy = "dlogits"
    for i in reversed(range(nl)):
        ops.append(Op("sum_rows", dict(M=dy, v="d:fc%d.b" % i)))     # AddBias.backward
        ready("fc%d.b" % i)
        ready("fc%d.W" % i)                                           # Matmul.backward (cuBLAS)
        if i > 0:
            g = tensor("fc%d.dgrad" % i, (B, dims[i]), "syn")        # dy @ W^T from cuBLAS
            dx = tensor("relu%d.dx" % (i - 1), (B, dims[i]), "grad")
            ops.append(Op("relu_bwd", dict(dy=g, x="relu%d.x" % (i - 1), dx=dx)))
            dy = dx
    ops.append(Op("sync_and_update", dict()))
    return dict(tensors=T, ops=ops, params=params, grad_order=order, batch=B)


def build_cnn_plan(batch=64, channels=32, num_classes=10):
    """Backward + update path of the small CNN of benchmark configuration 2:
    conv5x5(32)+bias -> ReLU -> maxpool2 -> conv5x5(32)+bias -> ReLU -> maxpool2
    -> linear 500 -> ReLU -> linear 10, on 1x28x28 inputs.  Convolution and
    matmul gradients are stand-ins; conv-bias and linear-bias gradients, ReLU /
    max-pool backward, softmax-CE and the update are computed."""
    T, ops, params, order = {}, [], [], []
    B, C = batch, channels

    def tensor(name, shape, kind):
        T[name] = Tensor(name, tuple(shape), kind)
        return name

    def param(name, shape):
        tensor(name, shape, "param")
        tensor("d:" + name, shape, "pgrad")
        params.append(name)

    def ready(p):
        order.append(p)
        ops.append(Op("grad_ready", dict(param=p)))

    param("conv1.W", (C, 1, 5, 5)); param("conv1.b", (C,))
    param("conv2.W", (C, C, 5, 5)); param("conv2.b", (C,))
    flat = C * 4 * 4
    param("fc1.W", (flat, 500)); param("fc1.b", (500,))
    param("fc2.W", (500, num_classes)); param("fc2.b", (num_classes,))
    tensor("relu1.x", (B, C, 24, 24), "act"); tensor("pool1.x", (B, C, 24, 24), "act")
    tensor("pool1.y", (B, C, 12, 12), "act")
    tensor("relu2.x", (B, C, 8, 8), "act"); tensor("pool2.x", (B, C, 8, 8), "act")
    tensor("pool2.y", (B, C, 4, 4), "act")
    tensor("relu3.x", (B, 500), "act")
    tensor("labels", (B,), "label")
    tensor("logits", (B, num_classes), "act")
    for n, shp in (("prob", (B, num_classes)), ("loss_vec", (B,)), ("loss", (1,)), ("dlogits", (B, num_classes))):
        tensor(n, shp, "grad")
    ops.append(Op("softmax", dict(x="logits", y="prob")))
    ops.append(Op("ce_fwd", dict(p="prob", t="labels", loss="loss_vec")))
    ops.append(Op("sum_all", dict(x="loss_vec", out="loss")))
    ops.append(Op("ce_bwd", dict(p="prob", t="labels", grad="dlogits")))
    ops.append(Op("scale", dict(x="dlogits", c=1.0 / B)))
    ops.append(Op("sum_rows", dict(M="dlogits", v="d:fc2.b"))); ready("fc2.b"); ready("fc2.W")
    g = tensor("fc2.dgrad", (B, 500), "syn")
    d3 = tensor("relu3.dx", (B, 500), "grad")
    ops.append(Op("relu_bwd", dict(dy=g, x="relu3.x", dx=d3)))
    ops.append(Op("sum_rows", dict(M=d3, v="d:fc1.b"))); ready("fc1.b"); ready("fc1.W")
    g = tensor("fc1.dgrad", (B, C, 4, 4), "syn")                      # reshaped dy @ W^T
    dp2 = tensor("pool2.dx", (B, C, 8, 8), "grad")
    ops.append(Op("maxpool_bwd", dict(x="pool2.x", y="pool2.y", dy=g, dx=dp2, kernel=(2, 2), stride=(2, 2), pad=(0, 0))))
    d2 = tensor("relu2.dx", (B, C, 8, 8), "grad")
    ops.append(Op("relu_bwd", dict(dy=dp2, x="relu2.x", dx=d2)))
    ops.append(Op("conv_bias_bwd", dict(dy=d2, db="d:conv2.b"))); ready("conv2.b"); ready("conv2.W")
    g = tensor("conv2.dgrad", (B, C, 12, 12), "syn")
    dp1 = tensor("pool1.dx", (B, C, 24, 24), "grad")
    ops.append(Op("maxpool_bwd", dict(x="pool1.x", y="pool1.y", dy=g, dx=dp1, kernel=(2, 2), stride=(2, 2), pad=(0, 0))))
    d1 = tensor("relu1.dx", (B, C, 24, 24), "grad")
    ops.append(Op("relu_bwd", dict(dy=dp1, x="relu1.x", dx=d1)))
    ops.append(Op("conv_bias_bwd", dict(dy=d1, db="d:conv1.b"))); ready("conv1.b"); ready("conv1.W")
    ops.append(Op("sync_and_update", dict()))
    return dict(tensors=T, ops=ops, params=params, grad_order=order, batch=B)
