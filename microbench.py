"""Per-kernel micro-benchmark of the backward-path kernels.

    python microbench.py bn --shape 32,256,56,56 [--relu] [--iters 20]
    python microbench.py relu --n 67108864
    python microbench.py maxpool --shape 32,64,112,112
    python microbench.py sgd | join | topk --n 100000000 | threshold --n ...

Each case allocates seeded inputs larger than L2 where the real workload's
are, launches the kernel through the C ABI and times it with CUDA events on
the launching stream (device time per call, averaged over ``--iters`` calls
issued back to back after ``--warmup`` calls).  It prints one line with the
algorithmic bytes, the time and the achieved GB/s.  The same command line is
what the ncu captures under ``profiles/`` were taken with.
"""
import argparse
import json
import sys

import torch

from singa_b200 import _lib
from singa_b200 import singa_wrap as sw


def timed(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def timed_graph(fn_of_stream, calls, reps=5):
    """Device time per call with no host in the loop: `calls` launches (the
    callee rotates its buffer sets so that inputs come from HBM, not L2) are
    captured into one CUDA graph; the best of `reps` replays is kept."""
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(calls):
            fn_of_stream(i, side.cuda_stream)          # eager warm-up (attribute calls, lazy init)
        side.synchronize()
        with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
            for i in range(calls):
                fn_of_stream(i, side.cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / calls
        best = t if best is None or t < best else best
    return best


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["bn", "relu", "join", "add_relu", "maxpool", "avgpool", "sgd",
                                     "pack", "threshold", "topk", "cast"])
    ap.add_argument("--shape", default="32,256,56,56")
    ap.add_argument("--n", type=int, default=1 << 26)
    ap.add_argument("--relu", action="store_true", help="bn: fused ReLU mask")
    ap.add_argument("--join", action="store_true", help="bn: fused gradient join + ReLU mask")
    ap.add_argument("--mode", default="compat", help="topk key: compat | magnitude")
    ap.add_argument("--argmax", action="store_true", help="maxpool: backward from the forward's arg-max record")
    ap.add_argument("--graph", action="store_true",
                    help="time a CUDA-graph replay of the calls (no host launch cost; same buffers every call)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    L = _lib.lib()
    torch.manual_seed(0)
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    shape = tuple(int(v) for v in a.shape.split(","))
    n = a.n

    if a.case == "bn":
        # Rotating buffer sets (together > 2x the 126 MB L2) inside one captured
        # graph: every call reads cold data and no host launch cost is timed.
        N, C, H, W = shape
        per_set = (5 if a.join else 4 if a.relu else 3) * 4 * N * C * H * W
        sets = max(2, -(-300 * 1024 * 1024 // per_set))
        mk = lambda scale=1.0: [torch.randn(shape, device=dev) * scale for _ in range(sets)]
        xs, dys, dxs = mk(), mk(1e-2), [torch.empty(shape, device=dev) for _ in range(sets)]
        rxs = mk() if (a.relu or a.join) else None
        dybs, jos = (mk(1e-2), [torch.empty(shape, device=dev) for _ in range(sets)]) if a.join else (None, None)
        sc, mu, r = torch.ones(C, device=dev), torch.zeros(C, device=dev), torch.ones(C, device=dev)
        ds, db = torch.empty(C, device=dev), torch.empty(C, device=dev)
        ws = torch.empty(max(L.sgb_bn_backward_workspace_bytes(N, C, H * W), 256), dtype=torch.uint8, device=dev)
        tail = (N, C, H * W, ws.data_ptr(), ws.numel())

        def fn_s(i, st):
            k = i % sets
            x, dy, dx = xs[k].data_ptr(), dys[k].data_ptr(), dxs[k].data_ptr()
            coef = (sc.data_ptr(), mu.data_ptr(), r.data_ptr())
            out = (dx, ds.data_ptr(), db.data_ptr())
            if a.join:
                _lib.call("sgb_bn_add_relu_backward_f32", x, dy, dybs[k].data_ptr(), rxs[k].data_ptr(), *coef,
                          jos[k].data_ptr(), *out, *tail, st)
            elif a.relu:
                _lib.call("sgb_bn_relu_backward_f32", x, dy, rxs[k].data_ptr(), *coef, *out, *tail, st)
            else:
                _lib.call("sgb_bn_backward_f32", x, dy, *coef, *out, *tail, st)

        nbytes = (24 if a.join else 16 if a.relu else 12) * N * C * H * W + 20 * C
        ms = timed_graph(fn_s, max(a.iters, 2 * sets))
        print(json.dumps({"case": "bn", "shape": a.shape, "fused_relu": bool(a.relu), "join": bool(a.join),
                          "buffer_sets": sets, "algorithmic_bytes": nbytes, "us": round(ms * 1e3, 2),
                          "GBps": round(nbytes / ms / 1e6, 1)}))
        return 0
    elif a.case in ("relu", "join", "add_relu", "cast"):
        x, y, z = (torch.randn(n, device=dev) for _ in range(3))
        out = torch.empty(n, device=dev)
        if a.case == "relu":
            fn = lambda: _lib.call("sgb_relu_backward_f32", y.data_ptr(), x.data_ptr(), out.data_ptr(), n, stream)
            nbytes = 12 * n
        elif a.case == "join":
            fn = lambda: _lib.call("sgb_binary_f32", 0, x.data_ptr(), y.data_ptr(), out.data_ptr(), n, stream)
            nbytes = 12 * n
        elif a.case == "add_relu":
            fn = lambda: _lib.call("sgb_add_relu_backward_f32", x.data_ptr(), y.data_ptr(), z.data_ptr(),
                                   out.data_ptr(), n, stream)
            nbytes = 16 * n
        else:
            h = torch.empty(n, device=dev, dtype=torch.float16)
            fn = lambda: _lib.call("sgb_cast_f32_f16", x.data_ptr(), h.data_ptr(), n, stream)
            nbytes = 6 * n
    elif a.case in ("maxpool", "avgpool"):
        x = torch.relu(torch.randn(shape, device=dev))
        if a.case == "maxpool":
            h = sw.CudnnPoolingHandle(x, (3, 3), (2, 2), (1, 1), True)
        else:
            h = sw.CudnnPoolingHandle(x, (shape[2], shape[3]), (1, 1), (0, 0), False)
        y = sw.GpuPoolingForward(h, x)
        dy, dx = torch.randn_like(y), torch.empty_like(x)
        if a.case == "maxpool" and a.argmax:
            _, arg = sw.GpuPoolingForwardArgmax(h, x)
            fn = lambda: _lib.call("sgb_maxpool_backward_argmax_f32", dy.data_ptr(), arg.data_ptr(), dx.data_ptr(),
                                   *h._geom(), stream)
            nbytes = 4 * (x.numel() + y.numel()) + y.numel()       # dy, record, dx
        elif a.case == "maxpool":
            fn = lambda: _lib.call("sgb_maxpool_backward_f32", x.data_ptr(), y.data_ptr(), dy.data_ptr(),
                                   dx.data_ptr(), *h._geom(), stream)
            nbytes = 4 * (2 * x.numel() + 2 * y.numel())
        else:
            fn = lambda: _lib.call("sgb_avgpool_backward_f32", dy.data_ptr(), dx.data_ptr(), *h._geom(), stream)
            nbytes = 4 * (x.numel() + y.numel())
    elif a.case in ("sgd", "pack"):
        from singa_b200.resnet50_path import build_plan, numel
        plan = build_plan()
        sizes = [numel(plan["tensors"][p].shape) for p in plan["params"]]
        ps = [torch.randn(k, device=dev) for k in sizes]
        gs = [torch.randn(k, device=dev) for k in sizes]
        ms = [torch.zeros(k, device=dev) for k in sizes]
        tot = sum(sizes)
        if a.case == "sgd":
            pp, sz, cnt = sw._ptr_table(ps)
            gp, mp = sw._ptr_table(gs)[0], sw._ptr_table(ms)[0]
            fn = lambda: _lib.call("sgb_sgd_update_multi_f32", pp, gp, mp, sz, cnt, 0.1, 0.9, 0.0, 1e-5, 0, 0.125, stream)
            nbytes = 20 * tot
        else:
            flat = torch.empty(tot, device=dev)
            pp, sz, cnt = sw._ptr_table(ps)
            fn = lambda: _lib.call("sgb_pack_f32", pp, sz, cnt, flat.data_ptr(), 0, stream)
            nbytes = 8 * tot
    else:  # threshold / topk on a flat gradient with residual
        g = torch.randn(n, device=dev) * 1e-3
        acc = torch.zeros(n, device=dev)
        idx = torch.empty(n, dtype=torch.int32, device=dev)
        val = torch.empty(n, device=dev)
        ws = torch.empty(L.sgb_sparse_workspace_bytes(n), dtype=torch.uint8, device=dev)
        if a.case == "threshold":
            nnz = torch.zeros(1, dtype=torch.int32, device=dev)
            fn = lambda: _lib.call("sgb_sparse_threshold_f32", g.data_ptr(), acc.data_ptr(), n, 2e-3, idx.data_ptr(),
                                   val.data_ptr(), nnz.data_ptr(), ws.data_ptr(), ws.numel(), stream)
        else:
            k = L.sgb_topk_count(0.01, n)
            mode = {"magnitude": 0, "compat": 1}[a.mode]
            fn = lambda: _lib.call("sgb_sparse_topk_f32", g.data_ptr(), acc.data_ptr(), None, n, k,
                                   mode, idx.data_ptr(), val.data_ptr(), ws.data_ptr(), ws.numel(), stream)
        nbytes = 12 * n

    if a.graph:
        def fn_s(i, st):
            nonlocal stream
            stream = st
            fn()
        ms = timed_graph(fn_s, a.iters)
    else:
        ms = timed(fn, a.iters, a.warmup)
    print(json.dumps({"case": a.case, "shape": a.shape if a.case in ("bn", "maxpool", "avgpool") else n,
                      "fused_relu": bool(a.relu), "algorithmic_bytes": nbytes, "us": round(ms * 1e3, 2),
                      "GBps": round(nbytes / ms / 1e6, 1)}))


if __name__ == "__main__":
    sys.exit(main())
