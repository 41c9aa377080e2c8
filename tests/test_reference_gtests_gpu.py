"""The reference's OWN unit tests on this repository's back end.  apache/singa's
test/singa/test_tensor_math.cc, test_tensor.cc and test_cross_entropy.cc (with
the loss layer it drives, src/model/loss/softmax_cross_entropy.cc) and its
vendored gtest are compiled unmodified (oracle/ref_cuda_build.py) and linked
once against the
reference's CUDA core and once against the same core with the replacement
tensor_math_cuda.h plugged in.  Every `*Cuda` case (tensor math on a CudaGPU
device: L2, Mult, row / column broadcasts, SumRows / SumColumns, strided Exp,
concatenation, row / column copies, RowMax, Broadcast, SoftPlus / SoftSign,
AsType; the loss layer's forward / backward with integer and array targets)
must pass on both; the Cpp cases ride along."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["reference", "sgb"])
def test_reference_unit_tests_pass(variant):
    from oracle import ref_cuda_build
    exe = ref_cuda_build.build_gtests(variant)
    if exe is None or not os.path.exists(exe):
        pytest.skip("the reference's gtest binary is not built (reference tree absent)")
    import torch
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    nccl = [os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), "nvidia", "nccl", "lib")]
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.pathsep.join([p for p in nccl + [libdir, env.get("LD_LIBRARY_PATH", "")] if p])
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    tail = r.stdout[-3000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    assert "[  PASSED  ]" in r.stdout and "FAILED" not in r.stdout, tail
    ran = [ln for ln in r.stdout.splitlines() if ln.startswith("[       OK ]")]
    assert sum("Cuda" in ln for ln in ran) >= 27, tail
