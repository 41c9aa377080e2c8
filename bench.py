"""Benchmark of the ResNet-50 backward + gradient-sync + update hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
                    [--dist-option plain|half] [--call-pattern]

One process per GPU (N > 1: launched by torch.distributed.run).  A step is one
pass of the hot path over one synthetic batch of 32 images per GPU: every
backward kernel the reference issues for ResNet-50 outside its cuDNN/cuBLAS
contractions, DistOpt's bucketed gradient all-reduce and the SGD-momentum
update.  Rank 0 prints ONE JSON line.

--impl reference times the CPU statement of the same path (the oracle, OpenMP
on all host cores) on a bounded sample of the workload.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "resnet50_backward_sync_update_images_per_sec"
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the batch-norm
# backward kernels, averaged per call over one step, from the ncu capture
# summarised in profiles/bench_resnet50_launch_list.md (fused / call-pattern plan).
NCU_BN_TRAFFIC_PER_CALL = {True: 71.8e6, False: 61.6e6}


def _traffic_from_summary():
    """Reads the two "... = X MB per call." lines of the committed launch-list
    summary (fused plan first, call-pattern plan second), so that the constant
    follows the capture; the literals above are the fallback."""
    import re
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles", "bench_resnet50_launch_list.md")
    try:
        found = re.findall(r"Batch-norm backward: \d+ calls, [\d.]+ MB of DRAM traffic per step = ([\d.]+) MB per call",
                           open(path).read())
        if len(found) == 2:
            return {True: float(found[0]) * 1e6, False: float(found[1]) * 1e6}
    except OSError:
        pass
    return NCU_BN_TRAFFIC_PER_CALL


BATCH = 32
CPU_SAMPLE_BATCH = 8


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(object):
    """nvidia-smi sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, "/tmp/sgb_clocks_%d.csv" % os.getpid()

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, reasons = [], set()
        try:
            for line in open(self.path):
                c = [v.strip() for v in line.split(",")]
                if len(c) < 9:
                    continue
                sm.append(float(c[1]))
                out["sm_max_mhz"] = float(c[2])
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def cpu_arm(steps, warmup, batch=CPU_SAMPLE_BATCH, threads=None):
    """The CPU statement of the hot path on a bounded sample: ResNet-50 at a
    reduced batch, on `threads` host threads (default: every core of the box,
    whatever OMP_NUM_THREADS the launcher exported).  Returns (images/s,
    ms/step, threads used)."""
    from oracle import build, cpu
    from oracle.path import OraclePath, make_tensors
    from singa_b200.resnet50_path import add_wgrad_refresh, build_plan
    build.build_oracle()
    cpu.set_num_threads(threads or os.cpu_count() or 1)
    plan = add_wgrad_refresh(build_plan(batch=batch, fused=False))
    tensors = make_tensors(plan, seed=0)
    ref = OraclePath(plan, tensors)
    for _ in range(warmup):
        ref.run_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        ref.run_step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return batch / dt, dt * 1e3, cpu.num_threads()


def config1_leg(torch, steps=50):
    """Benchmark configuration 1 (MLP 784-4096-4096-10, batch 256, SGD lr 0.05
    momentum 0.9), backward + update hot path without the contractions: the GPU
    executor (CUDA-graph replay, CUDA events) beside the reference's own
    lang::Cpp code - its tensor.cc / tensor_math_cpp.h compiled unmodified into
    oracle/_ref/libref_core.so - walking the same ops on the host cores."""
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import build_mlp_plan, fuse_plan
    plan = fuse_plan(build_mlp_plan())
    hp = HotPathGPU(plan, communicator=None, world=1, seed=0, lr=0.05, momentum=0.9, weight_decay=0.0)
    for _ in range(3):
        hp.run_step()
    torch.cuda.synchronize()
    g = hp.capture()
    for _ in range(10):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    gpu_ms = e0.elapsed_time(e1) / steps
    hp.release_graph()
    out = {"workload": "mlp_784_4096_4096_10_b256_backward_update", "steps": steps, "gpu_ms_per_step": gpu_ms,
           "gpu_images_per_sec": 256 / (gpu_ms / 1e3), "cpu_reference": None}
    try:
        from oracle import ref_core
        from oracle.path import make_tensors
        if not ref_core.available():
            raise ImportError("oracle/_ref/libref_core.so not built")
        raw = build_mlp_plan()
        t = make_tensors(raw, seed=0)
        dims = (784, 4096, 4096, 10)
        mlp = ref_core.MLP(256, dims, lr=0.05, momentum=0.9)
        for i in range(3):
            mlp.set(i, 0, t["fc%d.W" % i])
            mlp.set(i, 1, t["fc%d.b" % i])
        relu_x = [t["relu%d.x" % i] for i in range(2)]
        dgrad = [None] + [t["fc%d.dgrad" % i] for i in (1, 2)]
        wgrad = [t["d:fc%d.W" % i] for i in range(3)]
        ref_core.mlp_hot_path_step(mlp, t["logits"], t["labels"], relu_x, dgrad, wgrad)      # warm-up
        n = 5
        t0 = time.perf_counter()
        for _ in range(n):
            ref_core.mlp_hot_path_step(mlp, t["logits"], t["labels"], relu_x, dgrad, wgrad)
        ms = (time.perf_counter() - t0) / n * 1e3
        mlp.close()
        out["cpu_reference"] = {
            "kind": "reference", "ms_per_step": ms, "images_per_sec": 256 / (ms / 1e3), "cores": os.cpu_count(),
            "sample": "the full configuration-1 step, %d timed steps after 1 warm-up; the reference's elementwise "
                      "loops are serial (one core), only its BLAS-1 calls use OpenMP; includes the host copies "
                      "into singa::Tensor objects" % n}
    except Exception as e:      # the comparator is optional on a box without the prebuilt library
        out["cpu_reference_unavailable"] = str(e)[:200]
    return out


def reference_cuda_leg(torch, dist, path, rank, world, local, steps=10, warmup=2):
    """The same ResNet-50 backward + sync + update step on the reference's OWN
    CUDA / NCCL path, in the same run on the same GPUs: apache/singa's
    tensor.cc + tensor_math_cuda.h + math_kernel.cu, its cuDNN batch-norm /
    pooling operations and its unmodified communicator.cc, compiled from its
    sources into oracle/_ref/libref_singa_cuda.so (oracle/ref_cuda_build.py) and
    driven through its public C++ functions, one reference call per operation
    of the UNFUSED plan (its call pattern): ReLUBackward, `+=` joins,
    GpuBatchNormBackward / GpuPoolingBackward on their handles, SoftMax /
    CrossEntropyFwd / SumAll / SoftmaxCrossEntropyBwd / `/= N`, Sum(axis 0),
    DistOpt's bucket policy on Communicator::fusedSynch / synch / wait,
    `grad /= world` and the per-tensor Axpy chain of SGD.  Eager, like the
    reference (its operations are launched one by one from the host), timed
    with CUDA events on the default stream its kernels use.  The inputs are
    copies of this arm's tensors.  Returns None when the library is absent."""
    import ctypes as C
    lib_path = os.path.join(ROOT, "oracle", "_ref", "libref_singa_cuda.so")
    if not os.path.exists(lib_path):
        return None
    from singa_b200.opt import plan_buckets
    from singa_b200.resnet50_path import build_plan, numel
    L = C.CDLL(lib_path)
    for f in ("rs_tensor_new", "rs_relu_backward", "rs_add", "rs_sum_axis", "rs_sum_all", "rs_softmax",
              "rs_cross_entropy_fwd", "rs_softmax_cross_entropy_bwd", "rs_bn_handle_new", "rs_pool_handle_new",
              "rs_pool_backward", "rs_comm_new"):
        getattr(L, f).restype = C.c_void_p
    L.rs_init(local)
    plan = build_plan(batch=BATCH, fused=False)
    T = plan["tensors"]
    H = {}

    def new(shape, dtype=0):
        dims = (C.c_size_t * len(shape))(*shape)
        return C.c_void_p(L.rs_tensor_new(len(shape), dims, dtype))

    def put(name, h):
        old = H.get(name)
        if old is not None:
            L.rs_tensor_free(old)
        H[name] = h

    # inputs of the step: copies of this arm's device tensors
    for name, spec in T.items():
        if spec.kind in ("act", "stat", "syn", "param", "pgrad", "label"):
            src = path.t[name]
            h = new(spec.shape, 2 if spec.kind == "label" else 0)
            L.rs_tensor_from_device(h, C.c_void_p(src.data_ptr()), C.c_size_t(src.numel() * src.element_size()))
            H[name] = h
    for pname in plan["params"]:
        h = new(T[pname].shape)
        L.rs_tensor_set(h, C.c_float(0.0))
        H["m:" + pname] = h
    bn_handles, pool_handles = {}, {}
    for op in plan["ops"]:
        a = op.args
        if op.kind == "bn_bwd":
            bn_handles[a["x"]] = C.c_void_p(L.rs_bn_handle_new(C.c_float(0.9), H[a["x"]]))
        elif op.kind in ("maxpool_bwd", "avgpool_bwd"):
            key = a.get("x", a["dx"])
            if op.kind == "avgpool_bwd":      # the forward input only lends its shape to the handle
                H[a["dx"] + ".shape"] = new(T[a["dx"]].shape)
                H[a["dx"] + ".y"] = new(T[a["dy"]].shape)
                key = a["dx"] + ".shape"
            k, st, pd = a["kernel"], a["stride"], a["pad"]
            pool_handles[a["dx"]] = C.c_void_p(L.rs_pool_handle_new(H[key], k[0], k[1], st[0], st[1], pd[0], pd[1],
                                                                    1 if op.kind == "maxpool_bwd" else 0))
    comm = None
    if True:
        idb = C.create_string_buffer(L.rs_nccl_id_bytes())
        if rank == 0:
            L.rs_nccl_id_new(idb)
        if world > 1:
            box = [idb.raw if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            idb = C.create_string_buffer(box[0], len(box[0]))
        comm = C.c_void_p(L.rs_comm_new(local, world, idb, 4194304))
    order = plan["grad_order"]
    sizes = [numel(T["d:" + n].shape) for n in order]
    events = plan_buckets(sizes, 2097152)
    flush_after = {ev[1][-1]: ev for ev in events}
    index = {n: i for i, n in enumerate(order)}
    lr, mom, wd = C.c_float(0.1), C.c_float(0.9), C.c_float(1e-5)

    def step():
        for op in plan["ops"]:
            a, k = op.args, op.kind
            if k == "relu_bwd":
                put(a["dx"], C.c_void_p(L.rs_relu_backward(H[a["dy"]], H[a["x"]])))
            elif k == "add_out":
                put(a["out"], C.c_void_p(L.rs_add(H[a["a"]], H[a["b"]])))
            elif k == "bn_bwd":
                out = (C.c_void_p * 3)()
                L.rs_bn_backward(bn_handles[a["x"]], H[a["dy"]], H[a["x"]], H[a["scale"]], H[a["mean"]], H[a["invstd"]], out)
                put(a["dx"], C.c_void_p(out[0]))
                put(a["dscale"], C.c_void_p(out[1]))
                put(a["dbias"], C.c_void_p(out[2]))
            elif k == "maxpool_bwd":
                put(a["dx"], C.c_void_p(L.rs_pool_backward(pool_handles[a["dx"]], H[a["dy"]], H[a["x"]], H[a["y"]])))
            elif k == "avgpool_bwd":
                put(a["dx"], C.c_void_p(L.rs_pool_backward(pool_handles[a["dx"]], H[a["dy"]], H[a["dx"] + ".shape"],
                                                          H[a["dx"] + ".y"])))
            elif k == "softmax":
                put(a["y"], C.c_void_p(L.rs_softmax(H[a["x"]])))
            elif k == "ce_fwd":
                put(a["loss"], C.c_void_p(L.rs_cross_entropy_fwd(H[a["p"]], H[a["t"]])))
            elif k == "sum_all":
                put(a["out"], C.c_void_p(L.rs_sum_all(H[a["x"]])))
            elif k == "ce_bwd":
                put(a["grad"], C.c_void_p(L.rs_softmax_cross_entropy_bwd(H[a["p"]], H[a["t"]])))
            elif k == "scale":
                L.rs_div_scalar_inplace(H[a["x"]], C.c_float(BATCH))
            elif k == "sum_rows":
                put(a["v"], C.c_void_p(L.rs_sum_axis(H[a["M"]], 0)))
            elif k == "grad_ready":
                i = index[a["param"]]
                ev = flush_after.get(i)
                g = H["d:" + a["param"]]
                if ev is not None and ev[0] == "direct":
                    L.rs_comm_synch(comm, g)
                    continue
                one = (C.c_void_p * 1)(g)
                L.rs_comm_fused_synch(comm, one, 1, 0)
                if ev is not None:
                    arr = (C.c_void_p * len(ev[1]))(*[H["d:" + order[j]] for j in ev[1]])
                    L.rs_comm_fused_synch(comm, arr, len(ev[1]), 1)
            elif k == "sync_and_update":
                L.rs_comm_wait(comm)
                for pname in plan["params"]:
                    g = H["d:" + pname]
                    L.rs_div_scalar_inplace(g, C.c_float(world))
                    L.rs_sgd(H[pname], g, H["m:" + pname], lr, mom, wd)

    for _ in range(warmup):
        step()
    L.rs_sync()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    L.rs_sync()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / steps * 1e3
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        tt = torch.tensor([ms, wall], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, wall = float(tt[0]), float(tt[1])
    L.rs_comm_free(comm)
    return {"ms_per_step": ms, "host_ms_per_step": wall, "images_per_sec": BATCH * world / (ms / 1e3), "steps": steps,
            "mode": "eager (the reference launches one operation at a time), unfused call pattern, CUDA events",
            "library": "oracle/_ref/libref_singa_cuda.so: the reference's sources, compiled unmodified"}


def workload_config(world, dist_option, fused, use_graph, pool_argmax, relu_mask=False, threshold=2097152):
    """The `config` object shared by both arms (same keys, same values)."""
    return {"workload": "resnet50_b32_224_backward_sync_update", "batch_per_gpu": BATCH,
            "global_batch": BATCH * world, "dist_option": dist_option,
            "fusion": "bn+relu, join+relu, softmax+ce+grad" if fused else "none (one kernel per reference call)",
            "cuda_graph": use_graph, "pool_argmax_record": bool(pool_argmax), "relu_bit_mask": bool(relu_mask),
            "bucket_elems": 4194304, "threshold_elems": int(threshold),
            "excluded": "cuDNN/cuBLAS contractions (conv, linear): stand-in gradients, rewritten every step"}


def reference_main(args, rank, world):
    """The reference arm: the CPU statement of the path on the host cores of
    ONE box (rank 0 alone runs; the value is that of one host and is not
    multiplied by the number of GPUs).  Runs exactly --steps steps after
    --warmup warm-up steps on every core of the box; the per-step sample (the
    batch fed to the CPU) is halved from 8 until the whole run fits in about
    three minutes, and the sample actually used is reported."""
    if rank != 0:
        return
    steps, warmup = max(args.steps, 1), max(args.warmup, 0)
    batch = CPU_SAMPLE_BATCH
    _, probe_ms, _ = cpu_arm(1, 1, batch)                 # one timed step to size the run
    while batch > 1 and (steps + warmup) * probe_ms * batch / CPU_SAMPLE_BATCH > 180e3:
        batch //= 2
    v, ms, cores = cpu_arm(steps, warmup, batch)
    sample = "ResNet-50 hot path at batch %d (of %d) per step, fp32, %d OpenMP threads" % (batch, BATCH, cores)
    config = workload_config(world, args.dist_option, not args.call_pattern, not args.no_graph, args.pool_argmax,
                             args.relu_mask)
    config.update({"sample_batch": batch, "device": "host CPU, one box (value not scaled by n_gpus)",
                   "note": "CPU restatement (oracle port) of the reference path; the reference's own lang::Cpp "
                           "backend has no BatchNorm/Pooling without DNNL"})
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "images/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": v, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def percentiles(xs):
    xs = sorted(xs)

    def q(f):
        return xs[min(len(xs) - 1, int(round(f * (len(xs) - 1))))]
    return {"p10": round(q(0.1), 4), "p50": round(q(0.5), 4), "p90": round(q(0.9), 4), "max": round(xs[-1], 4)}


def sparse_leg(torch, dist, comm, rank, world, workload, n, K, W, sampler=None):
    """Sparse gradient exchange (benchmark configuration 5): every step each
    rank selects from a fresh flat gradient (plus its residual), all ranks
    exchange [index | value] payloads and every rank scatter-adds all payloads
    into the dense result.  Returns a dict (ms per exchange step = max over
    ranks, elements/s of the whole job, roofline of the step)."""
    multi = world > 1
    topk = workload == "sparse_topk"
    bounded = workload == "sparse_threshold_bounded"   # fixed exchange of 0.2 n slots, no host wait for the counts
    capacity = n // 5
    spars = 0.01 if topk else 2e-3
    fresh = min(K, 20)                       # distinct gradients held on the device (0.4 GB each at 1e8)
    gen = torch.Generator(device="cuda")
    grads = []
    for step in range(fresh):
        gen.manual_seed(20 * rank + step)
        grads.append(torch.randn(n, device="cuda", generator=gen) * 1e-3)
    work = torch.empty(n, device="cuda")
    acc = torch.zeros(n, device="cuda")

    def step(k):
        work.copy_(grads[k % fresh])         # the exchange overwrites its input with the dense result
        if bounded:
            comm.boundedSparsification([work], acc, spars, capacity)
        else:
            comm.sparsification(work, acc, spars, topk)
        comm.wait()

    def barrier():
        torch.cuda.synchronize()
        if multi:
            dist.barrier()

    for k in range(W):
        step(k)
    acc.zero_()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if sampler is not None:
        sampler.start()
    e0.record()
    for k in range(K):
        step(k)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / K
    if multi:
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if sampler is not None else None
    nnz = int((work != 0).sum().item())       # non-zeros of the last dense result
    # the copy of the fresh gradient is part of the loop but not of the exchange: time it alone
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for k in range(K):
        work.copy_(grads[k % fresh])
    c1.record()
    torch.cuda.synchronize()
    copy_ms = c0.elapsed_time(c1) / K
    peak, peak_kind = measured_peak()
    alg = 16.0 * n                            # read g, read acc, write acc, write dense result
    ex_ms = ms - copy_ms
    del grads, work, acc
    torch.cuda.empty_cache()
    return {"workload": workload, "elements_per_gpu": n, "spars": spars, "residual": True,
            "topk_mode": "compat" if topk else None, "steps": K, "warmup": W, "fresh_gradients": fresh,
            "ms_per_step": ex_ms, "elements_per_sec": n * world / (ex_ms / 1e3),
            "loop_ms_incl_gradient_copy": ms, "dense_nonzeros_after_last_step": nnz, "clocks": clocks,
            "capacity": capacity if bounded else None, "held_back": comm.sparseDropped() if bounded else None,
            "roofline": {"bound": "hbm", "achieved": round(alg / ex_ms / 1e6, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(alg / ex_ms / 1e6 / peak, 4), "peak_kind": peak_kind, "traffic": None,
                         "algorithmic_bytes_per_step": alg}}


def sparse_main(args, rank, world, local):
    """`--workload sparse_topk|sparse_threshold`: the sparse exchange alone, one JSON line."""
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("SGB_BENCH_WATCHDOG_S", "900")), exit=True)
    import torch
    import torch.distributed as dist
    from singa_b200 import _lib
    from singa_b200.communicator import Communicator, NcclIdHolder
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    _lib.lib()
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    box = [NcclIdHolder().id if rank == 0 else None]
    if multi:
        dist.broadcast_object_list(box, src=0)
    n = args.elements
    comm = Communicator(local, world, NcclIdHolder(box[0]), buffSize=n)
    K, W = max(args.steps, 1), max(args.warmup, 3)
    r = sparse_leg(torch, dist, comm, rank, world, args.workload, n, K, W,
                   sampler=ClockSampler(local) if rank == 0 else None)
    if rank == 0:
        print(json.dumps({
            "metric": "sparse_gradient_exchange_elements_per_sec", "value": r["elements_per_sec"],
            "unit": "elements/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {k: r[k] for k in ("workload", "elements_per_gpu", "spars", "residual", "topk_mode",
                                         "fresh_gradients", "loop_ms_incl_gradient_copy",
                                         "dense_nonzeros_after_last_step")},
            "clocks": r["clocks"], "roofline": r["roofline"],
        }), flush=True)
    torch.cuda.synchronize()
    comm.close()
    if multi:
        dist.barrier()
        dist.destroy_process_group()


def sync_check(torch, np, comm, rank, world):
    """Cross-rank value check of every dense synchronisation entry point on
    seeded per-rank buffers: every rank regenerates all ranks' inputs, so the
    expected sums are known locally.  fp32 sums within 1e-5, fp16 within 1e-3
    (relative to the largest expected magnitude)."""
    sizes = [1000003, 4096, 77, 250000, 1]            # odd sizes, a 1-element tensor, 1.25 M in total

    def inputs(r, tag):
        rng = np.random.default_rng(1000 * tag + r)
        return [rng.standard_normal(s).astype(np.float32) * np.float32(1e-2) for s in sizes]

    worst = {}

    def rel(got, want):
        want = np.asarray(want, np.float64)
        return float(np.abs(np.asarray(got, np.float64) - want).max() / max(np.abs(want).max(), 1e-30))

    def expect(tag, half=False):
        per_rank = [inputs(r, tag) for r in range(world)]
        if half:
            per_rank = [[a.astype(np.float16).astype(np.float64) for a in rr] for rr in per_rank]
        return [sum(per_rank[r][i].astype(np.float64) for r in range(world)) for i in range(len(sizes))]

    def dev(arrs, contiguous):
        if contiguous:
            flat = torch.from_numpy(np.concatenate(arrs)).cuda()
            out, off = [], 0
            for a in arrs:
                out.append(flat[off:off + a.size])
                off += a.size
            return out
        return [torch.from_numpy(np.concatenate([a, np.zeros(3, np.float32)])).cuda()[:a.size] for a in arrs]

    # synch: one tensor in place
    ts = dev(inputs(rank, 1), False)
    for t in ts:
        comm.synch(t)
    comm.wait()
    torch.cuda.synchronize()
    worst["synch"] = max(rel(t.cpu().numpy(), w) for t, w in zip(ts, expect(1)))
    # fusedSynch: contiguous list (reduced in place) and scattered list (packed)
    for name, contiguous, tag in (("fusedSynch_contiguous", True, 2), ("fusedSynch_scattered", False, 3)):
        ts = dev(inputs(rank, tag), contiguous)
        for t in ts:
            comm.fusedSynch([t], send=False)
        comm.fusedSynch(ts, send=True)
        comm.wait()
        torch.cuda.synchronize()
        worst[name] = max(rel(t.cpu().numpy(), w) for t, w in zip(ts, expect(tag)))
    # fp16 transport
    ts = dev(inputs(rank, 4), False)
    for t in ts:
        comm.fusedSynchHalf([t], send=False)
    comm.fusedSynchHalf(ts, send=True)
    comm.wait()
    torch.cuda.synchronize()
    worst["fusedSynchHalf"] = max(rel(t.cpu().numpy(), w) for t, w in zip(ts, expect(4, half=True)))
    ts = dev(inputs(rank, 5), False)
    comm.synchHalf(ts[0])
    comm.wait()
    torch.cuda.synchronize()
    worst["synchHalf"] = rel(ts[0].cpu().numpy(), expect(5, half=True)[0])
    tol = {"synch": 1e-5, "fusedSynch_contiguous": 1e-5, "fusedSynch_scattered": 1e-5,
           "fusedSynchHalf": 1e-3 * max(world, 2), "synchHalf": 1e-3 * max(world, 2)}
    ok = all(worst[k] <= tol[k] for k in worst)
    return worst, ok


def timeline(torch, path, comm):
    """One eager (uncaptured) step with every communicator phase and every
    per-bucket update bracketed by timing events on its own stream.  Returns
    rows per bucket: ms since the start of the step at which the bucket's last
    gradient was ready on the compute stream, its collective started / ended,
    its update ended; plus the end of the step."""
    path.profile = True
    for _ in range(2):                      # the first profiled step warms the event pools
        torch.cuda.synchronize()
        comm.profile_begin()
        path.run_step()
        comm.profile_mark("step_end")
        rows = comm.profile_end()
    path.profile = False
    buckets, cur = [], None
    step_end = None
    for name, t0, t1 in rows:
        if name == "bucket_ready":
            cur = {"ready": round(t0, 4)}
            buckets.append(cur)
        elif name == "step_end":
            step_end = round(t0, 4)
        elif cur is not None and name.startswith("Dist_s_"):
            cur["collective"] = name
            cur["start"], cur["end"] = round(t0, 4), round(t1, 4)
        elif cur is not None and name == "sgd_update_bucket":
            cur["update_end"] = round(t1, 4)
    coll_ms = sum(b["end"] - b["start"] for b in buckets if "end" in b)
    return {"mode": "eager, one step", "step_end_ms": step_end, "collective_ms_sum": round(coll_ms, 4),
            "buckets": buckets}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--dist-option", default="plain", choices=["plain", "half"])
    ap.add_argument("--call-pattern", action="store_true",
                    help="one kernel per reference call (no cross-op fusion)")
    ap.add_argument("--workload", default="resnet50", choices=["resnet50", "sparse_topk", "sparse_threshold", "sparse_threshold_bounded"],
                    help="resnet50 (headline) or the sparse gradient exchange microbench: a flat 1e8-element "
                         "fp32 gradient N(0, 1e-3^2), residual accumulation on, top-K ratio 0.01 / threshold 2e-3")
    ap.add_argument("--elements", type=int, default=100000000)
    ap.add_argument("--pool-argmax", action="store_true",
                    help="max-pool backward from the forward partner's arg-max record instead of (x, y): changes "
                         "what the backward consumes, so it is not the default")
    ap.add_argument("--relu-mask", action="store_true",
                    help="ReLU backward (alone or fused) from the forward partner's one-bit-per-element record "
                         "instead of the stored ReLU input: changes what the backward consumes, not the default")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-legs", action="store_true",
                    help="skip the fp16-sync and sparse-exchange legs that ride in the same JSON line")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="skip the leg that runs the reference's own CUDA / NCCL build of the same step")
    ap.add_argument("--nccl-max-ctas", type=int, default=16,
                    help="cap on the CTAs NCCL's kernels use at more than one GPU (ncclCommInitRankConfig maxCTAs; "
                         "0 = NCCL's default).  16 measured -1.7 %% step time at 2 GPUs, neutral at 4, -2.0 %% at 8: "
                         "fewer CTAs taken from the HBM-bound backward kernels while the collectives still hide")
    ap.add_argument("--no-register", action="store_true", help="do not register the gradient arena with NCCL")
    ap.add_argument("--threshold-elems", type=int, default=2097152,
                    help="DistOpt's threshold (python/singa/opt.py: backward_and_update): tensors above it are "
                         "reduced alone, smaller ones are staged and flushed once the bucket exceeds it; the "
                         "default is the reference's")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return reference_main(args, rank, world)
    if args.workload != "resnet50":
        return sparse_main(args, rank, world, local)

    import faulthandler
    # A rank that stops making progress ends itself with a traceback instead of
    # holding the GPUs until an outer time limit.
    faulthandler.dump_traceback_later(int(os.environ.get("SGB_BENCH_WATCHDOG_S", "900")), exit=True)
    import numpy as np
    import torch
    import torch.distributed as dist
    from singa_b200 import _lib
    from singa_b200.communicator import Communicator, NcclIdHolder
    from singa_b200.hot_path import HotPathGPU
    from singa_b200.resnet50_path import add_wgrad_refresh, algorithmic_bytes, build_plan, fuse_plan, mask_plan

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback "
                         "(use --impl reference for the CPU statement)")
    _lib.lib()
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        dist.init_process_group("gloo", rank=rank, world_size=world)

    def new_comm(buff, cap=True):
        box = [NcclIdHolder().id if rank == 0 else None]
        if multi:
            dist.broadcast_object_list(box, src=0)
        return Communicator(local, world, NcclIdHolder(box[0]), buffSize=buff,
                            max_ctas=args.nccl_max_ctas if (multi and cap) else 0)

    comm = new_comm(max(4194304, 2 * args.threshold_elems))   # a bucket holds at most threshold + one tensor <= threshold

    K, W = max(args.steps, 1), max(args.warmup, 3)
    WARM_REPLAYS = 10            # untimed graph replays (NCCL included) before the timed region, whatever W is
    fused = not args.call_pattern
    use_graph = not args.no_graph

    def make_path(dist_option, communicator):
        plan = build_plan(batch=BATCH, fused=False)        # the reference's call sequence ...
        if fused:
            plan = fuse_plan(plan)                         # ... rewritten by the peephole pass
        if args.relu_mask:
            plan = mask_plan(plan)                         # ReLU decisions from the forward partner's bit record
        plan = add_wgrad_refresh(plan)                     # the contractions' weight gradients are rewritten every step
        hp = HotPathGPU(plan, communicator=communicator, world=world, seed=1000 + rank, dist_option=dist_option,
                        pool_argmax=args.pool_argmax, threshold=args.threshold_elems)
        if multi and not args.no_register:
            communicator.register(hp.grad_arena)
        return plan, hp

    plan, path = make_path(args.dist_option, comm)
    by_family, nparam = algorithmic_bytes(plan, world, pool_argmax=args.pool_argmax)

    def barrier():
        torch.cuda.synchronize()
        if multi:
            dist.barrier()

    def max_over_ranks(v):
        if not multi:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_steps(hp, k_steps):
        """W eager warm-up steps, capture, warm replays, then exactly k_steps
        timed steps (own event pair each).  Returns (ms per step = max over
        ranks of the whole region / k_steps, per-step list of this rank, launches)."""
        launches = 0
        for _ in range(W):
            launches = hp.run_step()
        torch.cuda.synchronize()
        if use_graph:
            hp.capture()
            for _ in range(WARM_REPLAYS):
                hp.graph.replay()
            torch.cuda.synchronize()

        def one():
            if use_graph:
                hp.graph.replay()
            else:
                hp.run_step()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(k_steps + 1)]
        barrier()
        torch.cuda.profiler.start()     # lets `ncu --profile-from-start off` see exactly the timed steps
        marks[0].record()
        for i in range(k_steps):
            one()
            marks[i + 1].record()
        barrier()
        torch.cuda.profiler.stop()
        total = max_over_ranks(marks[0].elapsed_time(marks[-1])) / k_steps
        per = [marks[i].elapsed_time(marks[i + 1]) for i in range(k_steps)]
        return total, per, one, launches

    # ---- device-resident timing (clocks sampled from the warm replays to the end of the e2e region)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, per_step, one_step, _ = timed_steps(path, K)
    value = BATCH * world / (ms / 1e3)
    step_ms = percentiles(per_step)
    step_ms["max"] = round(max_over_ranks(step_ms["max"]), 4)

    # ---- end to end: pinned host batch + labels in, loss out, every step.
    # The next batch is prefetched on a copy stream while the current step runs
    # (two device slots); every step waits for its own batch, consumes its
    # labels, and the host reads that step's loss before going on.
    img_host = [torch.randn(BATCH, 3, 224, 224).pin_memory() for _ in range(2)]
    lab_host = [torch.randint(0, 1000, (BATCH,), dtype=torch.int32).pin_memory() for _ in range(2)]
    loss_host = torch.zeros(1).pin_memory()
    img_dev = [torch.empty_like(img_host[0], device="cuda") for _ in range(2)]
    lab_dev = [torch.empty_like(lab_host[0], device="cuda") for _ in range(2)]
    copy_stream = torch.cuda.Stream()
    arrived = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    main = torch.cuda.current_stream()

    def prefetch(k):
        slot = k % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])          # the step that used this slot is done with it
            img_dev[slot].copy_(img_host[slot], non_blocking=True)
            lab_dev[slot].copy_(lab_host[slot], non_blocking=True)
            arrived[slot].record(copy_stream)

    for ev in consumed:
        ev.record(main)
    barrier()
    t0 = time.perf_counter()
    prefetch(0)
    for k in range(K):
        slot = k % 2
        if k + 1 < K:
            prefetch(k + 1)
        main.wait_event(arrived[slot])
        path.t["labels"].copy_(lab_dev[slot], non_blocking=True)
        one_step()
        consumed[slot].record(main)
        loss_host.copy_(path.t["loss"], non_blocking=True)
        torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0) / K
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    e2e = {"value": BATCH * world / e2e_s, "unit": "images/s",
           "h2d_bytes_per_step": img_host[0].numel() * 4 + lab_host[0].numel() * 4, "d2h_bytes_per_step": 4,
           "ms_per_step": e2e_s * 1e3}

    # ---- per-family device times (instrumented eager pass, rank 0 reports)
    fam_ms = profile_families(path, torch)
    peak, peak_kind = measured_peak()
    fam = {}
    alias = {"relu_bwd": "relu_bwd", "relu_mask_bwd": "relu_mask_bwd", "add_relu_bwd": "add_relu_bwd",
             "add_relu_mask_bwd": "add_relu_mask_bwd", "add_out": "join", "bn_bwd": "bn_bwd",
             "bn_relu_bwd": "bn_relu_bwd", "bn_relu_mask_bwd": "bn_relu_mask_bwd",
             "bn_add_relu_bwd": "bn_add_relu_bwd", "maxpool_bwd": "maxpool_bwd",
             "avgpool_bwd": "avgpool_bwd", "wgrad_refresh": "wgrad_standin", "sgd": "sgd"}
    for k, name in alias.items():
        if k in fam_ms and name in by_family and fam_ms[k] > 0:
            gbs = by_family[name] / fam_ms[k] / 1e6
            fam[name] = {"ms": round(fam_ms[k], 4), "GBps": round(gbs, 1), "frac": round(gbs / peak, 3)}
    bn_keys = [k for k in ("bn_bwd", "bn_relu_bwd", "bn_relu_mask_bwd", "bn_add_relu_bwd") if k in fam_ms]
    bn_bytes = sum(by_family[k] for k in bn_keys)
    bn_ms = sum(fam_ms[k] for k in bn_keys)
    bn_launches = sum(1 for o in plan["ops"] if o.kind in bn_keys)
    achieved = bn_bytes / bn_ms / 1e6
    captured_plan = fused and not args.relu_mask
    roofline = {"bound": "hbm",
                "kernel": "batch-norm backward (cluster, streaming and channel-group kernels: all 53 calls)",
                "achieved": round(achieved, 1),
                "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "traffic": _traffic_from_summary()[fused] if (captured_plan or not fused) else None,
                "traffic_source": "ncu capture summarised in profiles/bench_resnet50_launch_list.md (a constant, "
                                  "not measured in this run)",
                "peak_kind": peak_kind, "launches_per_step": bn_launches,
                "algorithmic_bytes_per_launch": bn_bytes / max(bn_launches, 1),
                "avg_launch_ms": bn_ms / max(bn_launches, 1)}
    total_alg = sum(by_family.values())

    # ---- cross-rank value check and the eager per-bucket timeline (every rank runs them, rank 0 reports)
    worst, ok = sync_check(torch, np, comm, rank, world)
    ok = bool(max_over_ranks(0.0 if ok else 1.0) == 0.0)
    check = {"max_rel_err": {k: float("%.3e" % max_over_ranks(v)) for k, v in worst.items()}, "ok": ok,
             "tolerance": "1e-5 fp32, 1e-3 x world fp16, relative to the largest expected sum"}
    tl = timeline(torch, path, comm)
    launches_per_step = kernel_launches(path)
    # sticky fault word of the streaming batch-norm kernel (bounded waits between its CTAs): 0 on every rank
    import ctypes
    flags = ctypes.c_uint(0)
    _lib.call("sgb_bn_backward_faults", ctypes.byref(flags))
    bn_faults = int(max_over_ranks(float(flags.value)))
    if bn_faults:
        raise SystemExit("bench.py: the streaming batch-norm kernel recorded fault flags %d" % bn_faults)

    nvlink = None
    if multi:
        wire = 2.0 * (world - 1) / world * 4.0 * nparam * (0.5 if args.dist_option == "half" else 1.0)
        lower = wire / 900e9 * 1e3
        coll = tl["collective_ms_sum"]
        nvlink = {"bytes_per_step": wire, "formula": "2 (W-1)/W x gradient bytes, per GPU and direction",
                  "peak_GBps": 900.0, "peak_measured_GBps": 770.0, "lower_bound_ms": round(lower, 4),
                  "lower_bound_share_of_step": round(lower / ms, 4),
                  "collective_ms_sum": coll, "achieved_GBps": round(wire / coll / 1e6, 1) if coll else None,
                  "frac": round(wire / coll / 1e6 / 900.0, 4) if coll else None,
                  "frac_of_measured": round(wire / coll / 1e6 / 770.0, 4) if coll else None,
                  "note": "collective times from the eager timeline (they overlap the backward kernels)"}

    path.release_graph()          # graphs that captured NCCL work must go before the communicator
    import gc
    del one_step
    gc.collect()
    torch.cuda.synchronize()

    # ---- the reference's own CUDA / NCCL path on the same step, same GPUs, same run
    extra = {}
    if not args.no_extra_legs and not args.no_reference_cuda:
        try:
            rc = reference_cuda_leg(torch, dist, path, rank, world, local)
        except Exception as e:          # the comparator is optional
            rc = {"unavailable": str(e)[:200]}
        if rc is not None:
            if "ms_per_step" in rc:
                rc["ratio_vs_this_arm"] = rc["ms_per_step"] / ms
            extra["reference_cuda"] = rc
        gc.collect()
        torch.cuda.synchronize()

    # ---- configurations 4 and 5 with the same code, in the same line
    if not args.no_extra_legs and not args.call_pattern:
        other = "half" if args.dist_option == "plain" else "plain"
        K2 = min(K, 50)
        _, path2 = make_path(other, comm)
        ms2, per2, one2, _ = timed_steps(path2, K2)
        extra["config4_fp16_sync" if other == "half" else "config3_plain_sync"] = {
            "dist_option": other, "steps": K2, "ms_per_step": ms2, "images_per_sec": BATCH * world / (ms2 / 1e3),
            "step_ms": percentiles(per2)}
        path2.release_graph()
        del one2, path2
        gc.collect()
        torch.cuda.synchronize()
        del path
        gc.collect()
        torch.cuda.empty_cache()
        comm.close()
        comm = new_comm(args.elements, cap=False)     # bandwidth-bound payloads: NCCL's own CTA count
        legs = {}
        for wl in ("sparse_topk", "sparse_threshold", "sparse_threshold_bounded"):
            r = sparse_leg(torch, dist, comm, rank, world, wl, args.elements, 20, 3)
            legs[wl] = {k: r[k] for k in ("spars", "topk_mode", "steps", "ms_per_step", "elements_per_sec",
                                          "dense_nonzeros_after_last_step", "roofline", "capacity", "held_back")}
            if multi and wl == "sparse_topk":      # all-gather: every GPU receives the (W-1) payloads of its peers
                pay = 8.0 * _lib.lib().sgb_topk_count(r["spars"], args.elements)
                legs[wl]["nvlink_lower_bound_ms"] = round((world - 1) * pay / 900e9 * 1e3, 5)
        extra["config5_sparse_exchange"] = dict(legs, elements_per_gpu=args.elements, fresh_gradients=20)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, cms, cores = cpu_arm(steps=3, warmup=1)
        cpu_baseline = {"value": v, "unit": "images/s", "cores": cores, "kind": "port",
                        "sample": "ResNet-50 hot path at batch %d (of %d), 3 timed steps after 1 warm-up, "
                                  "oracle C port, %d OpenMP threads" % (CPU_SAMPLE_BATCH, BATCH, cores),
                        "ms_per_step": cms}

    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.no_extra_legs:
        extra["config1_mlp"] = config1_leg(torch)

    if rank == 0:
        config = workload_config(world, args.dist_option, fused, use_graph, args.pool_argmax, args.relu_mask,
                                 args.threshold_elems)
        config.update({"l2": "inputs larger than L2: %.1f GB touched per step vs 126 MB" % (total_alg / 1e9),
                       "algorithmic_GB_per_step": round(total_alg / 1e9, 3),
                       "hot_path_GBps": round(total_alg / ms / 1e6, 1),
                       "warm_graph_replays": WARM_REPLAYS if use_graph else 0,
                       "nccl_max_ctas": args.nccl_max_ctas if multi else 0, "arena_registered": bool(multi and not args.no_register)})
        line = {
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms, "step_ms": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * K,
            "roofline": roofline, "roofline_by_family": fam, "sync_check": check, "bn_faults": bn_faults,
            "nvlink": nvlink,
            "timeline": tl, "cpu_baseline": cpu_baseline,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    comm.close()
    if multi:
        dist.barrier()
        dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()


def kernel_launches(path):
    """Kernels of this library launched per step (NCCL's own are not counted).
    Batch-norm backward is one launch, except when a channel (x and dy of all
    samples) exceeds what a cluster of eight CTAs can stage (8 x 100 KB): then
    it is the reduce + apply pair."""
    per = {"sgb_relu_backward_f32": 1, "sgb_add_relu_backward_f32": 1, "sgb_binary_f32": 1,
           "sgb_relu_backward_mask_f32": 1, "sgb_add_relu_backward_mask_f32": 1,
           "sgb_maxpool_backward_f32": 1, "sgb_maxpool_backward_argmax_f32": 1,
           "sgb_avgpool_backward_f32": 1, "sgb_softmax_rows_f32": 1, "sgb_cross_entropy_f32": 1,
           "sgb_sum_all_f32": 1, "sgb_softmax_cross_entropy_bwd_f32": 1,
           "sgb_softmax_cross_entropy_grad_f32": 1, "sgb_softmax_cross_entropy_fused_f32": 1,
           "sgb_scalar_f32": 1, "sgb_sum_rows_f32": 1, "sgb_set_f32": 1}
    n = 0
    for name, args in path.calls:
        if name in ("sgb_bn_backward_f32", "sgb_bn_relu_backward_f32", "sgb_bn_relu_backward_mask_f32",
                    "sgb_bn_add_relu_backward_f32"):
            N, _, HW = args[-6:-3]          # (..., N, C, HW, workspace, workspace bytes, stream)
            n += 2 if N * HW * 8 > 8 * 100 * 1024 else 1
        elif name == "sgb_unpack_f32":       # stand-in weight gradients: one launch per 72 tensors
            n += (args[4] + 71) // 72
        else:
            n += per.get(name, 0)
    if path.comm is not None:
        for kind, idx in path.events:
            if kind == "fused" and path.dist_option == "half":
                n += 2 * ((len(idx) + 71) // 72)  # pack+cast and unpack+cast launches at flush
            # fp32 buckets are contiguous arena slices: reduced in place, no pack / unpack
            elif path.dist_option == "half":
                n += 2                           # cast down, cast up
    if getattr(path, "update_on_arrival", False):
        n += sum((len(idx) + 71) // 72 for _, idx in path.events)   # one fused SGD group per bucket
    else:
        n += (len(path.plan["params"]) + 71) // 72               # one fused SGD group per step
    return n


def profile_families(path, torch, reps=5):
    """Device time per op family.  All calls of one family are captured, in
    step order, into one CUDA graph (no host gaps, no other kernels between
    them) and the replay is timed with CUDA events on the replaying stream;
    the best of `reps` replays is kept.  Inputs are the buffers the preceding
    full steps left behind, i.e. far larger than L2 in total."""
    import numpy as np
    L = path.lib
    kinds = [o.kind for o in path.plan["ops"]]
    fams = {}
    for (name, args), kind in zip(path.calls, kinds):
        if name == "grad_ready":
            continue
        fams.setdefault("sgd" if name == "sync_and_update" else kind, []).append((name, args))
    out = {}
    side = torch.cuda.Stream()
    for fam, calls in fams.items():
        def issue(stream):
            for name, args in calls:
                if name == "sync_and_update":
                    pp, gp, mp, sizes, n = path.sgd_tables
                    L.sgb_sgd_update_multi_f32(pp, gp, mp, sizes, n, path.lr, path.momentum, 0.0,
                                               path.weight_decay, 0,
                                               float(np.float32(1.0) / np.float32(path.world)), stream)
                else:
                    getattr(L, name)(*[stream if v == "STREAM" else v for v in args])
        g = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                issue(side.cuda_stream)
        torch.cuda.current_stream().wait_stream(side)
        g.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            t = a.elapsed_time(b)
            best = t if best is None or t < best else best
        out[fam] = best
    return out


if __name__ == "__main__":
    main()
