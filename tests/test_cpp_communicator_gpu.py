"""The C++ mirrors of singa::Communicator (include/sgb_communicator.hpp) and of
the operation handles (include/sgb_operations.hpp) driven from a C++ program
on one GPU.  Communicator, world size 1: every public method runs, and a
one-rank exchange must return its input (all-reduce of one rank, fp16 round
trip of fp16-exact values, top-K with ratio 1, threshold 0).  Operations: the
reference's own max-pooling vectors (test_cudnn_pooling.cc) and closed-form
batch-norm / conv-bias cases on the input of its BN API test."""
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
#include "sgb_operations.hpp"

static float* to_dev(const std::vector<float>& h) {
  float* d;
  cudaMalloc(&d, (h.size() ? h.size() : 1) * sizeof(float));
  cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice);
  return d;
}
static bool near(const float* dev, const std::vector<float>& want, float tol, const char* what) {
  std::vector<float> got(want.size());
  cudaMemcpy(got.data(), dev, want.size() * sizeof(float), cudaMemcpyDeviceToHost);
  for (size_t i = 0; i < want.size(); ++i)
    if (std::fabs(got[i] - want[i]) > tol) { std::printf("%s[%zu]: %g vs %g\n", what, i, got[i], want[i]); return false; }
  return true;
}

static bool operations() {
  bool ok = true;
  // max pooling: the reference's vectors
  const std::vector<float> px = {POOL_X}, py = {POOL_Y}, pdy = {POOL_DY}, pdx = {POOL_DX};
  sgb::CudnnPoolingHandle ph({1, 1, 3, 3}, {2, 2}, {1, 1}, {0, 0}, true);
  float *x = to_dev(px), *y = to_dev(py), *dy = to_dev(pdy), *dx = to_dev(pdx);
  cudaMemset(y, 0, py.size() * sizeof(float));
  cudaMemset(dx, 0, pdx.size() * sizeof(float));
  sgb::GpuPoolingForward(ph, x, y, nullptr);
  sgb::GpuPoolingBackward(ph, dy, x, y, dx, nullptr);
  ok = ok && near(y, py, 0.f, "pool y") && near(dx, pdx, 0.f, "pool dx");
  // batch norm on the BN API test's input: mean (5.5, 11), inverse std (1/4.5, 1/9); with dy = 1
  // everywhere dbias = 8, dscale = 0 and dx = 0
  const std::vector<float> bx = {BN_X}, ones(16, 1.0f), two(2, 1.0f), zero2(2, 0.0f);
  sgb::CudnnBatchNormHandle bh(0.1f, {2, 2, 2, 2});
  void* ws;
  cudaMalloc(&ws, bh.workspace_bytes() + 256);
  float *bxd = to_dev(bx), *byd = to_dev(ones), *sc = to_dev(two), *bi = to_dev(zero2), *rm = to_dev(zero2),
        *rv = to_dev(two), *mean = to_dev(zero2), *var = to_dev(zero2), *g = to_dev(ones), *bdx = to_dev(ones),
        *ds = to_dev(two), *db = to_dev(two);
  sgb::GpuBatchNormForwardTraining(bh, bxd, sc, bi, rm, rv, byd, mean, var, ws, bh.workspace_bytes(), nullptr);
  ok = ok && near(mean, {5.5f, 11.0f}, 1e-6f, "bn mean") && near(var, {1.0f / 4.5f, 1.0f / 9.0f}, 1e-6f, "bn invstd");
  ok = ok && near(rm, {0.55f, 1.1f}, 1e-6f, "running mean");
  sgb::GpuBatchNormBackward(bh, g, bxd, sc, mean, var, bdx, ds, db, ws, bh.workspace_bytes(), nullptr);
  ok = ok && near(db, {8.0f, 8.0f}, 0.f, "dbias") && near(ds, {0.0f, 0.0f}, 1e-5f, "dscale") &&
       near(bdx, std::vector<float>(16, 0.0f), 1e-6f, "bn dx");
  // conv bias gradient of dy = 1: N * H * W per channel
  sgb::GpuConvBackwardb(g, db, 2, 2, 2, 2, ws, bh.workspace_bytes(), nullptr);
  ok = ok && near(db, {8.0f, 8.0f}, 0.f, "conv db");
  return ok && cudaDeviceSynchronize() == cudaSuccess;
}

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
  ok = ok && operations();
  std::printf(ok ? "ok\n" : "FAILED\n");
  return ok ? 0 : 1;
}
'''


def test_cpp_communicator_world_1_and_operation_mirrors(tmp_path, golden):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not available on this box")
    import torch
    from singa_b200 import build
    lib_path = build.build()
    libdir = os.path.dirname(lib_path)
    src, exe = tmp_path / "comm.cu", tmp_path / "comm"
    lit = lambda v: ", ".join("%rf" % float(a) for a in v)
    pool, bn = golden["maxpool_cudnn"], golden["batchnorm_training_api"]
    program = PROGRAM
    for key, vals in (("POOL_X", pool["x"]), ("POOL_Y", pool["y"]), ("POOL_DY", pool["dy"]), ("POOL_DX", pool["dx"]),
                      ("BN_X", bn["x"])):
        program = program.replace("{" + key + "}", "{" + lit(vals) + "}")
    src.write_text(program)
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
