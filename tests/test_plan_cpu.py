"""Host-side logic without a GPU: the ResNet-50 hot-path plan, the bucket
policy against the oracle's restatement, top-K count arithmetic."""
import numpy as np

from oracle import comm as ocomm
from singa_b200.opt import plan_buckets
from singa_b200.resnet50_path import algorithmic_bytes, build_plan, fuse_plan, numel


def test_resnet50_plan_sizes():
    plan = build_plan()
    T = plan["tensors"]
    assert len(plan["params"]) == 161
    assert sum(numel(T[p].shape) for p in plan["params"]) == 25557032
    kinds = [o.kind for o in plan["ops"]]
    assert kinds.count("bn_bwd") == 53 and kinds.count("relu_bwd") == 49 and kinds.count("add_out") == 16
    by, nparam = algorithmic_bytes(plan)
    assert by["relu_bwd"] == 12 * 307478528                    # 307.5 M ReLU elements per step
    assert abs(by["bn_bwd"] - 12 * 355.6e6) < 0.01e9
    assert by["maxpool_bwd"] == 4 * (2 * 25690112 + 2 * 6422528)
    assert sorted(plan["grad_order"]) == sorted(plan["params"])


def test_bucket_policy_matches_oracle_and_reference_counts():
    plan = build_plan()
    sizes = [numel(plan["tensors"]["d:" + n].shape) for n in plan["grad_order"]]
    ev = plan_buckets(sizes)
    assert ev == ocomm.plan_buckets(sizes)
    assert sum(1 for k, _ in ev if k == "direct") == 3          # the three 2,359,296-element 3x3 convs
    assert sum(1 for k, _ in ev if k == "fused") == 8
    first = ev[0]
    assert first[0] == "fused" and len(first[1]) == 5 and sum(sizes[i] for i in first[1]) == 3101672
    for k, idx in ev:
        tot = sum(sizes[i] for i in idx)
        assert tot <= 4194304                                    # fits buffSize
        if k == "direct":
            assert tot > 2097152
    rng = np.random.default_rng(0)
    for _ in range(20):
        s = rng.integers(1, 3000000, rng.integers(1, 40)).tolist()
        assert plan_buckets(s) == ocomm.plan_buckets(s)


def test_fused_plan_has_same_parameters_and_fewer_passes():
    a, b = build_plan(fused=False), build_plan(fused=True)
    assert a["params"] == b["params"] and a["grad_order"] == b["grad_order"]
    assert sum(algorithmic_bytes(b)[0].values()) < sum(algorithmic_bytes(a)[0].values())


def test_oracle_topk_modes():
    s = np.array([0.5, -2.5, 0.1, 2.4, -0.7, 3.0, 0.0, -2.0], np.float32)
    assert ocomm.topk_select(s, 3, "magnitude").tolist() == [1, 3, 5]
    # the reference comparator truncates to int first: keys 0,2,0,2,0,3,0,2
    assert ocomm.topk_select(s, 3, "compat").tolist() == [1, 3, 5]
    assert ocomm.topk_select(s, 2, "compat").tolist() == [1, 5]          # tie 2.5/2.4 -> lower index
    assert ocomm.topk_select(s * 0.1, 3, "compat").tolist() == [0, 1, 2]  # everything ties at 0
    assert ocomm.topk_count(0.01, 100000000) == 1000000


def test_peephole_pass_reproduces_the_hand_fused_plan():
    def key(plan):
        return [(o.kind, sorted((k, str(v)) for k, v in o.args.items())) for o in plan["ops"]]
    for kw in (dict(), dict(batch=4, image=64, num_classes=10, blocks=(2, 1, 1, 1))):
        by_hand = build_plan(fused=True, **kw)
        by_pass = fuse_plan(build_plan(fused=False, **kw))
        assert key(by_hand) == key(by_pass)
        assert set(by_pass["tensors"]) == set(by_hand["tensors"])
        by_hand = build_plan(fused=True, join_bn=True, **kw)
        by_pass = fuse_plan(build_plan(fused=False, **kw), join_bn=True)
        assert key(by_hand) == key(by_pass)
        assert any(o.kind == "bn_add_relu_bwd" for o in by_pass["ops"])
        assert not any(o.kind == "add_relu_bwd" for o in by_pass["ops"])
    # an intermediate with a second reader must not be fused away
    from singa_b200.resnet50_path import Op
    plan = build_plan(batch=2, image=64, num_classes=10, blocks=(1, 1, 1, 1))
    ops = list(plan["ops"])
    i = next(k for k, o in enumerate(ops) if o.kind == "relu_bwd" and ops[k + 1].kind == "bn_bwd"
             and ops[k + 1].args["dy"] == o.args["dx"])
    extra = Op("sum_all", dict(x=ops[i].args["dx"], out="loss"))
    fused = fuse_plan(dict(plan, ops=ops[:i + 2] + [extra] + ops[i + 2:]))
    assert any(o.kind == "relu_bwd" and o.args["dx"] == ops[i].args["dx"] for o in fused["ops"])


def test_traffic_totals_and_idempotent_fusion():
    call = build_plan(fused=False)
    fused = fuse_plan(call)
    gb = lambda p: sum(algorithmic_bytes(p)[0].values()) / 1e9
    assert abs(gb(call) - 10.898) < 1e-3 and abs(gb(fused) - 8.4635) < 1e-3
    again = fuse_plan(fused)
    assert [o.kind for o in again["ops"]] == [o.kind for o in fused["ops"]]
    kinds = [o.kind for o in fused["ops"]]
    assert kinds.count("softmax_ce") == 1 and "softmax" not in kinds and "ce_fwd" not in kinds
    assert kinds.count("bn_relu_bwd") == 33 and kinds.count("bn_bwd") == 20 and kinds.count("add_relu_bwd") == 15


def test_loss_head_is_not_fused_across_a_use_of_the_gradient():
    from singa_b200.resnet50_path import Op
    plan = build_plan(batch=2, image=64, num_classes=10, blocks=(1, 1, 1, 1))
    ops = list(plan["ops"])
    i = next(k for k, o in enumerate(ops) if o.kind == "ce_fwd")
    # an op between the loss and the gradient that reads the gradient buffer blocks the rewrite
    blocker = Op("sum_all", dict(x="dlogits", out="loss"))
    fused = fuse_plan(dict(plan, ops=ops[:i + 1] + [blocker] + ops[i + 1:]))
    kinds = [o.kind for o in fused["ops"]]
    assert "softmax_ce" not in kinds and "softmax" in kinds and "ce_grad" in kinds


def test_join_relu_bn_chain_without_a_second_reader_keeps_every_read_produced():
    """add_out(a, b -> t) ; relu_bwd(t, r -> m) ; bn_bwd(m): `m` has one reader,
    so the first rule rewrites the ReLU into add_relu_bwd; the batch-norm rule
    must then see the REWRITTEN producer and leave the pair alone (or fold it
    through the join rule) - never read a tensor nothing produces."""
    from singa_b200.resnet50_path import READS, WRITES, Op, Tensor
    shape = (2, 8, 4, 4)
    T = {n: Tensor(n, shape, "syn") for n in ("a", "b")}
    T.update({n: Tensor(n, shape, "act") for n in ("r", "x")})
    T.update({n: Tensor(n, shape, "grad") for n in ("t", "m", "dx")})
    for n in ("scale", "mean", "invstd", "ds", "db"):
        T[n] = Tensor(n, (8,), "stat")
    ops = [Op("add_out", dict(a="a", b="b", out="t")),
           Op("relu_bwd", dict(dy="t", x="r", dx="m")),
           Op("bn_bwd", dict(dy="m", x="x", scale="scale", mean="mean", invstd="invstd", dx="dx",
                             dscale="ds", dbias="db"))]
    base = dict(tensors=T, ops=ops, params=[], grad_order=[], batch=2)
    for join_bn in (False, True):
        plan = fuse_plan(base, join_bn=join_bn)
        produced = set()
        for op in plan["ops"]:
            for key in READS[op.kind]:
                name = op.args[key]
                assert name in plan["tensors"], (join_bn, op.kind, name)
                assert name in produced or plan["tensors"][name].kind in ("syn", "act", "stat"), (op.kind, name)
            produced.update(op.args[k] for k in WRITES[op.kind])
        kinds = [o.kind for o in plan["ops"]]
        assert kinds == (["bn_add_relu_bwd"] if join_bn else ["add_relu_bwd", "bn_bwd"]), kinds
        assert "dx" in produced


def test_every_collective_of_a_step_is_ordered_after_the_compute_stream():
    """Replays the bucket events of the ResNet-50 step through the
    communicator's edge planner (the same function the GPU code emits its
    events from) for each synchronisation option: every collective must be
    ordered after the compute stream AT ITS OWN CALL (directly, or through the
    pre-processing stream), the next bucket's collective must not wait for
    the stream that carries the previous bucket's update, and wait() must join
    exactly the streams that received work."""
    import ctypes as C

    from singa_b200 import _lib
    lib = _lib.lib()
    plan = build_plan()
    sizes = [numel(plan["tensors"]["d:" + n].shape) for n in plan["grad_order"]]
    events = plan_buckets(sizes)
    assert len(events) == 11
    E = dict(compute_c1=1, compute_s=2, c1_s=4, c2done_s=8, s_c1=16, s_c2=32, s_compute=64, c1_compute=128,
             c2_compute=256, mark_c2=512)

    def call(state, kind):
        edges, res = (C.c_uint * 4)(), C.c_int()
        assert lib.sgb_comm_order_plan(state, kind, edges, C.byref(res)) == 0
        return list(edges), res.value

    for option, kinds in (("plain/arena", {"direct": 0, "fused": 1}), ("plain/packed", {"direct": 0, "fused": 2}),
                          ("half", {"direct": 4, "fused": 3})):
        state = (C.c_ubyte * 4)()
        n_compute_edges = 0
        for ev_kind, _ in events:
            (pre, before, after, post), result = call(state, kinds[ev_kind])
            direct = bool(before & E["compute_s"])
            via_c1 = bool(pre & E["compute_c1"]) and bool(before & E["c1_s"])
            assert direct or via_c1, (option, ev_kind)
            n_compute_edges += 1
            if option == "plain/arena":
                assert before == E["compute_s"], "in-place buckets wait for the compute stream only"
                assert result == 2 and after & E["s_c2"]
            if option == "half":
                assert result == 2 and after & E["s_c2"] and post & E["mark_c2"]
        assert n_compute_edges == len(events)
        (_, join, _, _), _ = call(state, 7)
        want = E["s_compute"] | (E["c1_compute"] if option != "plain/arena" else 0) | \
            (E["c2_compute"] if option != "plain/packed" else 0)
        if option == "plain/packed":
            want |= E["c2_compute"]       # the direct tensors' results are consumed on c2
        assert join == want, (option, join, want)
        assert list(state) == [0, 0, 0, 0]
        (_, join, _, _), _ = call(state, 7)
        assert join == 0                  # nothing to join after a wait
    assert lib.sgb_comm_order_plan(None, 0, None, None) == -1
    state, edges = (C.c_ubyte * 4)(), (C.c_uint * 4)()
    assert lib.sgb_comm_order_plan(state, 8, edges, None) != 0
