"""The C++ mirror of singa::Communicator (include/sgb_communicator.hpp) driven
from a C++ program on one GPU (world size 1): every public method runs, and a
one-rank exchange must return its input (all-reduce of one rank, fp16 round
trip of fp16-exact values, top-K with ratio 1, threshold 0)."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r'''
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include <vector>
#include "sgb_communicator.hpp"

static bool same(const float* dev, const std::vector<float>& want) {
  std::vector<float> got(want.size());
  cudaMemcpy(got.data(), dev, want.size() * sizeof(float), cudaMemcpyDeviceToHost);
  for (size_t i = 0; i < want.size(); ++i)
    if (got[i] != want[i]) { std::printf("mismatch at %zu: %g vs %g\n", i, got[i], want[i]); return false; }
  return true;
}

int main() {
  const size_t n = 100003;
  std::vector<float> h(n);
  for (size_t i = 0; i < n; ++i) h[i] = static_cast<float>(static_cast<int>(i % 257) - 128) * 0.25f;   // fp16-exact
  float *a, *b, *acc;
  cudaMalloc(&a, n * sizeof(float));
  cudaMalloc(&b, n * sizeof(float));
  cudaMalloc(&acc, 2 * n * sizeof(float));
  auto reset = [&] {
    cudaMemcpy(a, h.data(), n * sizeof(float), cudaMemcpyHostToDevice);
    cudaMemcpy(b, h.data(), n * sizeof(float), cudaMemcpyHostToDevice);
    cudaMemset(acc, 0, 2 * n * sizeof(float));
  };
  sgb::NcclIdHolder id;
  sgb::Communicator c(0, 1, id, 4 * n);
  if (c.world_size != 1 || c.global_rank != 0 || c.local_rank != 0) return 2;
  sgb::TensorRef ta{a, n, false}, tb{b, n, false};
  bool ok = true;
  reset();
  c.synch(ta, nullptr);
  c.wait(nullptr);
  ok = ok && same(a, h);
  c.fusedSynch({ta}, nullptr, false);
  c.fusedSynch({tb}, nullptr, false);
  c.fusedSynch({ta, tb}, nullptr, true);
  c.wait(nullptr);
  ok = ok && same(a, h) && same(b, h);
  c.synchHalf(ta, nullptr);
  c.fusedSynchHalf({tb}, nullptr, false);
  c.fusedSynchHalf({tb}, nullptr, true);
  c.wait(nullptr);
  ok = ok && same(a, h) && same(b, h);
  c.sparsification(ta, acc, 1.0f, true, nullptr);                 // top-K of everything
  c.wait(nullptr);
  ok = ok && same(a, h);
  c.fusedSparsification({ta, tb}, nullptr, 0.0f, false, nullptr);  // threshold 0 keeps every non-zero
  c.wait(nullptr);
  ok = ok && same(a, h) && same(b, h);
  if (cudaDeviceSynchronize() != cudaSuccess) return 3;
  std::printf(ok ? "ok\n" : "FAILED\n");
  return ok ? 0 : 1;
}
'''


def test_cpp_communicator_world_1(tmp_path):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not available on this box")
    import torch
    from singa_b200 import build
    lib_path = build.build()
    libdir = os.path.dirname(lib_path)
    src, exe = tmp_path / "comm.cu", tmp_path / "comm"
    src.write_text(PROGRAM)
    r = subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                        os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir, "-lsgb",
                        "-Xlinker", "-rpath=" + libdir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    extra = [os.path.join(os.path.dirname(torch.__file__), "lib")]
    try:
        import nvidia.nccl
        extra.append(os.path.join(list(nvidia.nccl.__path__)[0], "lib"))
    except Exception:
        pass
    env = dict(os.environ, LD_LIBRARY_PATH=":".join(extra + [os.environ.get("LD_LIBRARY_PATH", "")]))
    out = subprocess.run([str(exe)], capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), (out.returncode, out.stdout, out.stderr)
