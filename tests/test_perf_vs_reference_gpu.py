"""Device time of the new kernels against the reference's own CUDA path on the
same B200, at the ResNet-50 shapes that dominate a step: the reference's
unmodified launchers (oracle/_ref/libref_cuda.so) and the cuDNN calls it
issues for batch-norm / pooling backward (oracle/_ref/libref_cudnn.so).

Every case rotates over buffer sets larger than L2 and is timed from a
CUDA-graph replay (no host launch cost on either side), best of 5.  The test
fails if a new kernel is slower than the call it replaces; the measured times
are written to $SGB_PERF_OUT (JSON) when that variable is set."""
import ctypes as C
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_CUDA = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
REF_CUDNN = os.path.join(ROOT, "oracle", "_ref", "libref_cudnn.so")
RESULTS = {}


def p(t):
    return C.c_void_p(t.data_ptr())


@pytest.fixture(scope="module")
def libs():
    if not (os.path.exists(REF_CUDA) and os.path.exists(REF_CUDNN)):
        pytest.skip("oracle/_ref checker libraries not built")
    from singa_b200 import _lib
    try:
        rd = C.CDLL(REF_CUDNN)
    except OSError as e:
        pytest.skip("cuDNN not loadable: %s" % e)
    rd.refcudnn_bn_min_epsilon.restype = C.c_double
    return _lib.lib(), C.CDLL(REF_CUDA), rd


def graph_time(call, sets, reps=5):
    """call(k, stream): one launch on buffer set k.  Returns microseconds per call."""
    calls = 2 * sets
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(sets):
            call(i, C.c_void_p(side.cuda_stream))         # eager warm-up (lazy initialisation)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
            for i in range(calls):
                call(i % sets, C.c_void_p(side.cuda_stream))
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
        t = e0.elapsed_time(e1) * 1e3 / calls
        best = t if best is None or t < best else best
    return best


def n_sets(bytes_per_set):
    return max(2, -(-320 * 1024 * 1024 // bytes_per_set))


def record(name, ours, ref, alg_bytes, margin):
    RESULTS[name] = {"ours_us": round(ours, 2), "reference_us": round(ref, 2), "speedup": round(ref / ours, 2),
                     "ours_GBps": round(alg_bytes / ours / 1e3, 1), "reference_GBps": round(alg_bytes / ref / 1e3, 1)}
    out = os.environ.get("SGB_PERF_OUT")
    if out:
        with open(out, "w") as f:
            json.dump(RESULTS, f, indent=1)
    assert ours <= margin * ref, "%s: %.1f us vs reference %.1f us" % (name, ours, ref)


@pytest.mark.parametrize("op", ["relubackward", "add"])
def test_elementwise_not_slower_than_reference_launcher(libs, op):
    L, rc, _ = libs
    n = 32 * 64 * 112 * 112                                 # the largest ReLU of ResNet-50
    sets = n_sets(12 * n)
    a = [torch.randn(n, device="cuda") for _ in range(sets)]
    b = [torch.randn(n, device="cuda") for _ in range(sets)]
    o = [torch.empty(n, device="cuda") for _ in range(sets)]
    if op == "relubackward":
        ours = graph_time(lambda k, s: L.sgb_relu_backward_f32(p(a[k]), p(b[k]), p(o[k]), n, s), sets)
        ref = graph_time(lambda k, s: rc.ref_relubackward(C.c_size_t(n), p(a[k]), p(b[k]), p(o[k]), s), sets)
    else:
        ours = graph_time(lambda k, s: L.sgb_binary_f32(0, p(a[k]), p(b[k]), p(o[k]), n, s), sets)
        ref = graph_time(lambda k, s: rc.ref_add(C.c_size_t(n), p(a[k]), p(b[k]), p(o[k]), s), sets)
    record(op + "_25.7M", ours, ref, 12 * n, 1.05)


# every distinct batch-norm shape of ResNet-50 at batch 32
@pytest.mark.parametrize("shape", [(32, 64, 112, 112), (32, 64, 56, 56), (32, 256, 56, 56), (32, 128, 56, 56),
                                   (32, 128, 28, 28), (32, 512, 28, 28), (32, 256, 28, 28), (32, 256, 14, 14),
                                   (32, 1024, 14, 14), (32, 512, 14, 14), (32, 512, 7, 7), (32, 2048, 7, 7)])
def test_batchnorm_backward_not_slower_than_cudnn(libs, shape):
    L, _, rd = libs
    N, Cc, H, W = shape
    n = N * Cc * H * W
    sets = n_sets(12 * n)
    x = [torch.randn(shape, device="cuda") for _ in range(sets)]
    dy = [torch.randn(shape, device="cuda") * 1e-2 for _ in range(sets)]
    dx = [torch.empty(shape, device="cuda") for _ in range(sets)]
    sc, mu, r = torch.ones(Cc, device="cuda"), torch.zeros(Cc, device="cuda"), torch.ones(Cc, device="cuda")
    ds, db = torch.empty(Cc, device="cuda"), torch.empty(Cc, device="cuda")
    ws = torch.empty(max(L.sgb_bn_backward_workspace_bytes(N, Cc, H * W), 256), dtype=torch.uint8, device="cuda")
    eps = C.c_double(rd.refcudnn_bn_min_epsilon())
    ours = graph_time(lambda k, s: L.sgb_bn_backward_f32(p(x[k]), p(dy[k]), p(sc), p(mu), p(r), p(dx[k]), p(ds), p(db),
                                                         N, Cc, H * W, p(ws), ws.numel(), s), sets)
    ref = graph_time(lambda k, s: rd.refcudnn_bn_backward(0, N, Cc, H, W, eps, p(x[k]), p(dy[k]), p(sc), p(mu), p(r),
                                                          p(dx[k]), p(ds), p(db), s), sets)
    record("bn_backward_%dx%dx%dx%d" % shape, ours, ref, 12 * n + 20 * Cc, 1.0)


def test_pooling_backward_not_slower_than_cudnn(libs):
    L, _, rd = libs
    for name, shape, k, s_, pd, is_max in (("maxpool_backward_stem", (32, 64, 112, 112), 3, 2, 1, 1),
                                           ("avgpool_backward_head", (32, 2048, 7, 7), 7, 1, 0, 0)):
        N, Cc, H, W = shape
        OH, OW = (H + 2 * pd - k) // s_ + 1, (W + 2 * pd - k) // s_ + 1
        nx, ny = N * Cc * H * W, N * Cc * OH * OW
        sets = n_sets(8 * nx + 8 * ny)
        x = [torch.relu(torch.randn(shape, device="cuda")) for _ in range(sets)]
        y = [torch.empty(N, Cc, OH, OW, device="cuda") for _ in range(sets)]
        dy = [torch.randn(N, Cc, OH, OW, device="cuda") for _ in range(sets)]
        dx = [torch.empty(shape, device="cuda") for _ in range(sets)]
        args = (N, Cc, H, W, OH, OW, k, k, pd, pd, s_, s_)
        for i in range(sets):
            assert rd.refcudnn_pooling(0, is_max, *args, p(x[i]), p(y[i]), None, None, None) == 0
        torch.cuda.synchronize()
        geo = (N, Cc, H, W, k, k, pd, pd, s_, s_)
        if is_max:
            ours = graph_time(lambda q, s: L.sgb_maxpool_backward_f32(p(x[q]), p(y[q]), p(dy[q]), p(dx[q]), *geo, s), sets)
            alg = 4 * (2 * nx + 2 * ny)
        else:
            ours = graph_time(lambda q, s: L.sgb_avgpool_backward_f32(p(dy[q]), p(dx[q]), *geo, s), sets)
            alg = 4 * (nx + ny)
        ref = graph_time(lambda q, s: rd.refcudnn_pooling(1, is_max, *args, p(x[q]), p(y[q]), p(dy[q]), p(dx[q]), s), sets)
        record(name, ours, ref, alg, 1.0)


def test_topk_selection_not_slower_than_reference_sort(libs):
    """Top-K selection step of the sparse exchange at the benchmark size: the
    reference generates indices and sorts all 10^8 (value, index) pairs
    (communicator.cc:741-750 -> generateindex, sortbykey); the new path selects
    with a three-pass radix select.  Event-timed, eager (Thrust allocates)."""
    L, rc, _ = libs
    n = 100000000
    k = L.sgb_topk_count(0.01, n)
    g = torch.randn(n, device="cuda") * 1e-3
    acc = torch.zeros(n, device="cuda")
    idx, val = torch.empty(n, dtype=torch.int32, device="cuda"), torch.empty(n, device="cuda")
    ws = torch.empty(L.sgb_sparse_workspace_bytes(n), dtype=torch.uint8, device="cuda")

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) * 1e3
            best = t if best is None or t < best else best
        return best

    ours = timed(lambda: L.sgb_sparse_topk_f32(p(g), p(acc), None, n, k, 1, p(idx), p(val), p(ws), ws.numel(),
                                               None), 5)
    key = torch.empty(n, device="cuda")

    def reference():
        key.copy_(g)
        rc.ref_generateindex(C.c_size_t(n), p(idx), None)
        rc.ref_sortbykey(C.c_size_t(n), p(key), p(idx), None)

    ref = timed(reference, 2)
    record("topk_select_1e8_k1e6", ours, ref, 12 * n, 1.0)
