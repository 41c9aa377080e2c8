"""The replacement back end on the reference's OWN types.  apache/singa's
Tensor / Device / Scheduler sources are compiled twice (oracle/ref_cuda_build.py):
with its own CUDA back end, and with this repository's tensor_math_cuda.h,
operation adapters and Communicator adapter plugged in at its build-time
plug-in points.  A fixed battery of singa::Tensor operations - elementwise ops
on dense and transposed views, reductions, the loss head, casts, the optimizer's
Axpy chain, cuBLAS contractions, GpuBatchNormBackward / GpuPoolingBackward on
their handle classes, and every Communicator mode at one rank - runs through
each build in its own process; the results must agree: bit for bit where the
arithmetic is elementwise, within 1e-5 (fp32) / 1e-3 (fp16 transport) where a
reduction order or a library differs."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

EXACT = {"relu", "relu_backward", "add", "sub", "eltwise_mult", "div", "add_transposed_left", "add_transposed_right",
         "mul_both_transposed", "compare_0", "compare_1", "compare_2", "compare_3", "compare_4", "scalar_chain",
         "cross_entropy", "softmax_ce_bwd", "f32_f16_f32", "f32_i32_f32", "row_max", "comm_synch", "comm_fused_a",
         "comm_fused_b", "maxpool_y", "maxpool2_y", "maxpool2_dx", "unary_5", "unary_6", "unary_7",
         "comm_topk_dense", "comm_topk_residual", "row_column_ops"}
HALF = {"comm_fused_half_a", "comm_fused_half_b", "comm_synch_half"}


@pytest.fixture(scope="module")
def results(tmp_path_factory):
    from oracle import ref_cuda_build
    for v in ("reference", "sgb"):
        if ref_cuda_build.build_variant(v) is None or not os.path.exists(ref_cuda_build.LIBS[v]):
            pytest.skip("the CUDA core variants are not built (reference tree absent)")
    out = {}
    d = tmp_path_factory.mktemp("singa_core")
    for v in ("reference", "sgb"):
        path = str(d / (v + ".npz"))
        r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "singa_core_worker.py"), v, path],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, "%s worker failed:\n%s\n%s" % (v, r.stdout[-2000:], r.stderr[-4000:])
        out[v] = dict(np.load(path))
    return out


def test_every_result_of_the_battery_agrees(results):
    ref, got = results["reference"], results["sgb"]
    assert set(ref) <= set(got)
    assert len(ref) > 70
    for name in sorted(ref):
        a, b = ref[name].astype(np.float64), got[name].astype(np.float64)
        assert a.shape == b.shape, name
        assert np.isfinite(b).all(), name
        if name in EXACT:
            assert np.array_equal(ref[name], got[name]), "%s differs (max %.3e)" % (name, np.abs(a - b).max())
            continue
        tol = 1e-3 if name in HALF else 1e-5
        scale = max(np.abs(a).max(), 1e-30)
        assert np.abs(a - b).max() <= tol * scale, "%s: rel %.3e" % (name, np.abs(a - b).max() / scale)


def test_conv_bias_gradient_on_singa_tensors(results):
    got = results["sgb"]
    want = got["conv_bias_backward_want"].astype(np.float64)
    assert np.abs(got["conv_bias_backward"] - want).max() <= 1e-5 * np.abs(want).max()


def test_one_rank_synchronisation_is_the_identity(results):
    """At one rank every dense mode must return its input (fp16 transport: its
    rounding), and top-K must move exactly K entries out of the residual."""
    got = results["sgb"]
    assert np.array_equal(got["comm_synch"], got["comm_fused_a"])
    k = int(np.ceil(np.float32(0.01) * 200000))
    assert int((got["comm_topk_dense"] != 0).sum()) == k
    both = (got["comm_topk_dense"] != 0) & (got["comm_topk_residual"] != 0)
    assert not both.any()
