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
NCU_BN_TRAFFIC_PER_CALL = {True: 77.8e6, False: 65.5e6}
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


def cpu_arm(steps, warmup, batch=CPU_SAMPLE_BATCH):
    """The CPU statement of the hot path on a bounded sample: ResNet-50 at a
    reduced batch, all host threads.  Returns (images/s, ms/step, cores)."""
    from oracle import build, cpu
    from oracle.path import OraclePath, make_tensors
    from singa_b200.resnet50_path import build_plan
    build.build_oracle()
    plan = build_plan(batch=batch, fused=False)
    tensors = make_tensors(plan, seed=0)
    ref = OraclePath(plan, tensors)
    for _ in range(warmup):
        ref.run_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        ref.run_step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return batch / dt, dt * 1e3, cpu.num_threads()


def reference_main(args, rank, world):
    """The reference arm: the CPU statement of the path on the host cores.  Runs
    exactly --steps steps after --warmup warm-up steps; the per-step sample (the
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
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "images/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "resnet50_b32_224_backward_sync_update", "device": "host CPU",
                   "note": "CPU restatement (oracle port) of the reference path; the reference's own lang::Cpp "
                           "backend has no BatchNorm/Pooling without DNNL"},
        "cpu_baseline": {"value": v, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def sparse_main(args, rank, world, local):
    """Sparse gradient exchange: every step each rank selects from a fresh flat
    gradient (plus its residual), all ranks exchange [index | value] payloads
    and every rank scatter-adds all payloads into the dense result.  One JSON
    line: steps/s of the whole job, per-step time (max over ranks), payload."""
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
    topk = args.workload == "sparse_topk"
    spars = 0.01 if topk else 2e-3
    K, W = max(args.steps, 1), max(args.warmup, 3)
    fresh = min(K, 20)                       # distinct gradients held on the device (0.4 GB each)
    gen = torch.Generator(device="cuda")
    grads = []
    for step in range(fresh):
        gen.manual_seed(20 * rank + step)
        grads.append(torch.randn(n, device="cuda", generator=gen) * 1e-3)
    work = torch.empty(n, device="cuda")
    acc = torch.zeros(n, device="cuda")

    def step(k):
        work.copy_(grads[k % fresh])         # the exchange overwrites its input with the dense result
        comm.sparsification(work, acc, spars, topk)
        comm.wait()

    def barrier():
        torch.cuda.synchronize()
        if multi:
            dist.barrier()

    for k in range(W):
        step(k)
    acc.zero_()
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if rank == 0:
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
    clocks = sampler.stop() if rank == 0 else None
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
    if rank == 0:
        print(json.dumps({
            "metric": "sparse_gradient_exchange_elements_per_sec", "value": n * world / (ex_ms / 1e3),
            "unit": "elements/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ex_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "elements_per_gpu": n, "spars": spars, "residual": True,
                       "topk_mode": "compat" if topk else None, "fresh_gradients": fresh,
                       "loop_ms_incl_gradient_copy": ms, "dense_nonzeros_after_last_step": nnz,
                       "l2": "inputs larger than L2: 0.4 GB per operand"},
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": round(alg / ex_ms / 1e6, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(alg / ex_ms / 1e6 / peak, 4), "peak_kind": peak_kind, "traffic": None,
                         "algorithmic_bytes_per_step": alg},
        }), flush=True)
    torch.cuda.synchronize()
    comm.close()
    if multi:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--dist-option", default="plain", choices=["plain", "half"])
    ap.add_argument("--call-pattern", action="store_true",
                    help="one kernel per reference call (no cross-op fusion)")
    ap.add_argument("--workload", default="resnet50", choices=["resnet50", "sparse_topk", "sparse_threshold"],
                    help="resnet50 (headline) or the sparse gradient exchange microbench: a flat 1e8-element "
                         "fp32 gradient N(0, 1e-3^2), residual accumulation on, top-K ratio 0.01 / threshold 2e-3")
    ap.add_argument("--elements", type=int, default=100000000)
    ap.add_argument("--pool-argmax", action="store_true",
                    help="max-pool backward from the forward partner's arg-max record instead of (x, y): changes "
                         "what the backward consumes, so it is not the default")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    from singa_b200.resnet50_path import add_wgrad_refresh, algorithmic_bytes, build_plan, fuse_plan

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback "
                         "(use --impl reference for the CPU statement)")
    _lib.lib()
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    box = [NcclIdHolder().id if rank == 0 else None]
    if multi:
        dist.broadcast_object_list(box, src=0)
    comm = Communicator(local, world, NcclIdHolder(box[0]), buffSize=4194304)

    K, W = max(args.steps, 1), max(args.warmup, 3)
    fused = not args.call_pattern
    plan = build_plan(batch=BATCH, fused=False)        # the reference's call sequence ...
    if fused:
        plan = fuse_plan(plan)                         # ... rewritten by the peephole pass
    plan = add_wgrad_refresh(plan)                     # the contractions' weight gradients are rewritten every step
    path = HotPathGPU(plan, communicator=comm, world=world, seed=1000 + rank, dist_option=args.dist_option,
                      pool_argmax=args.pool_argmax)
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

    # ---- warm-up (eager), graph capture, warm replays
    launches = 0
    for _ in range(W):
        launches = path.run_step()
    torch.cuda.synchronize()
    use_graph = not args.no_graph
    if use_graph:
        path.capture()
        path.graph.replay()
        torch.cuda.synchronize()

    def one_step():
        if use_graph:
            path.graph.replay()
        else:
            path.run_step()

    # ---- device-resident timing
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if rank == 0:
        sampler.start()
    torch.cuda.profiler.start()     # lets `ncu --profile-from-start off` see exactly the timed steps
    e0.record()
    for _ in range(K):
        one_step()
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1)) / K
    value = BATCH * world / (ms / 1e3)

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
    alias = {"relu_bwd": "relu_bwd", "add_relu_bwd": "add_relu_bwd", "add_out": "join", "bn_bwd": "bn_bwd",
             "bn_relu_bwd": "bn_relu_bwd", "bn_add_relu_bwd": "bn_add_relu_bwd", "maxpool_bwd": "maxpool_bwd", "avgpool_bwd": "avgpool_bwd", "sgd": "sgd"}
    for k, name in alias.items():
        if k in fam_ms and name in by_family and fam_ms[k] > 0:
            gbs = by_family[name] / fam_ms[k] / 1e6
            fam[name] = {"ms": round(fam_ms[k], 4), "GBps": round(gbs, 1), "frac": round(gbs / peak, 3)}
    bn_keys = [k for k in ("bn_bwd", "bn_relu_bwd", "bn_add_relu_bwd") if k in fam_ms]
    bn_bytes = sum(by_family[k] for k in bn_keys)
    bn_ms = sum(fam_ms[k] for k in bn_keys)
    bn_launches = sum(1 for o in plan["ops"] if o.kind in bn_keys)
    achieved = bn_bytes / bn_ms / 1e6
    roofline = {"bound": "hbm", "kernel": "batch-norm backward (reduce + apply)", "achieved": round(achieved, 1),
                "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "traffic": NCU_BN_TRAFFIC_PER_CALL[fused],
                "peak_kind": peak_kind, "launches_per_step": bn_launches,
                "algorithmic_bytes_per_launch": bn_bytes / max(bn_launches, 1),
                "avg_launch_ms": bn_ms / max(bn_launches, 1)}
    total_alg = sum(by_family.values())

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, cms, cores = cpu_arm(steps=3, warmup=1)
        cpu_baseline = {"value": v, "unit": "images/s", "cores": cores, "kind": "port",
                        "sample": "ResNet-50 hot path at batch %d (of %d), 3 timed steps after 1 warm-up, "
                                  "oracle C port, %d OpenMP threads" % (CPU_SAMPLE_BATCH, BATCH, cores),
                        "ms_per_step": cms}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "resnet50_b32_224_backward_sync_update", "batch_per_gpu": BATCH,
                       "global_batch": BATCH * world, "dist_option": args.dist_option,
                       "fusion": "bn+relu, join+relu, softmax+ce+grad" if fused else "none (one kernel per reference call)",
                       "cuda_graph": use_graph, "pool_argmax_record": bool(args.pool_argmax), "bucket_elems": 4194304, "threshold_elems": 2097152,
                       "l2": "inputs larger than L2: %.1f GB touched per step vs 126 MB" % (total_alg / 1e9),
                       "excluded": "cuDNN/cuBLAS contractions (conv, linear): stand-in gradients",
                       "algorithmic_GB_per_step": round(total_alg / 1e9, 3),
                       "hot_path_GBps": round(total_alg / ms / 1e6, 1)},
            "clocks": clocks, "e2e": e2e, "gpu_launches": kernel_launches(path) * K,
            "roofline": roofline, "roofline_by_family": fam, "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    path.release_graph()          # graphs that captured NCCL work must go before the communicator
    import gc
    gc.collect()
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
           "sgb_maxpool_backward_f32": 1, "sgb_maxpool_backward_argmax_f32": 1,
           "sgb_avgpool_backward_f32": 1, "sgb_softmax_rows_f32": 1, "sgb_cross_entropy_f32": 1,
           "sgb_sum_all_f32": 1, "sgb_softmax_cross_entropy_bwd_f32": 1,
           "sgb_softmax_cross_entropy_grad_f32": 1, "sgb_softmax_cross_entropy_fused_f32": 1,
           "sgb_scalar_f32": 1, "sgb_sum_rows_f32": 1}
    n = 0
    for name, args in path.calls:
        if name in ("sgb_bn_backward_f32", "sgb_bn_relu_backward_f32", "sgb_bn_add_relu_backward_f32"):
            N, _, HW = args[-6:-3]          # (..., N, C, HW, workspace, workspace bytes, stream)
            n += 2 if N * HW * 8 > 8 * 100 * 1024 else 1
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
