"""The C-ABI library loads without a GPU and exports every symbol that
include/sgb.h declares (no compute calls here)."""
import ctypes

import torch  # noqa: F401  (loads torch's NCCL before libsgb.so binds to libnccl.so.2)

from singa_b200 import _lib, build


def test_library_builds_and_exports_all_declared_symbols():
    path = build.build()
    handle = ctypes.CDLL(path)
    decls = _lib.declarations()
    assert len(decls) > 20
    missing = [name for name, _, _ in decls if not hasattr(handle, name)]
    assert not missing, missing


def test_status_strings_and_version():
    lib = _lib.lib()
    assert lib.sgb_version() >= 100
    assert lib.sgb_status_string(0) == b"ok"
    for code in range(-9, 0):
        assert lib.sgb_status_string(code) != b"unknown status"


def test_argument_validation_needs_no_gpu():
    # NULL pointers and bad enums are rejected on the host before any launch.
    lib = _lib.lib()
    assert lib.sgb_relu_backward_f32(None, None, None, 0, None) == 0      # n == 0 is a no-op
    assert lib.sgb_relu_backward_f32(None, None, None, 16, None) == -1    # SGB_ERR_NULL
    assert lib.sgb_binary_f32(99, 1, 1, 1, 0, None) in (0, -6)


def test_launcher_library_exports_the_reference_symbols():
    """libsgb_singa.so defines the `singa::cuda::*` launchers under exactly the
    mangled names the reference's math_kernel.cu exports (list extracted from
    the compiled reference, tests/golden/make_golden.py): all 75 of them."""
    import os
    import subprocess
    build.build()
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "golden", "singa_cuda_launcher_symbols.txt")) as f:
        want = set(f.read().split())
    assert len(want) == 75
    rows = subprocess.run(["nm", "-D", "--defined-only", build.ADAPTER_LIB], capture_output=True, text=True,
                          check=True).stdout
    have = set(r.split()[2] for r in rows.splitlines() if "_ZN5singa4cuda" in r)
    assert not (want - have), sorted(want - have)
    assert not (have - want), sorted(have - want)
    ctypes.CDLL(build.ADAPTER_LIB)       # resolves libsgb.so through its $ORIGIN runpath


def test_cpp_headers_compile_link_and_run(tmp_path):
    """include/sgb_communicator.hpp and include/sgb_operations.hpp (the C++
    mirrors of singa::Communicator and of the batch-norm / pooling / conv-bias
    operation handles and functions) compile warning-free as C++17 without CUDA
    headers, everything instantiates, and the program links against libsgb.so.
    The run checks the handles' size arithmetic and asks for the size of the
    NCCL id (no GPU)."""
    import os
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        import pytest
        pytest.skip("g++ not available")
    lib_path = build.build()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "use_communicator.cc"
    src.write_text(r'''
#include "sgb_communicator.hpp"
#include "sgb_operations.hpp"
int main(int argc, char**) {
  // handle arithmetic needs no GPU: the reference's own size rules
  sgb::CudnnBatchNormHandle bn(0.9f, {32, 64, 56, 56}), bn2(0.9f, {16, 100});
  sgb::CudnnPoolingHandle mp({32, 64, 112, 112}, {3, 3}, {2, 2}, {1, 1}, true);
  if (bn.is_2d || !bn2.is_2d || bn2.height != 1 || bn.height * bn.width != 3136) return 3;
  if (mp.pooled_height != 56 || mp.pooled_width != 56 || !mp.is_max_pooling) return 4;
  if (argc > 1) {   // instantiated for the compiler and linker only: needs a GPU and its NCCL peers to run
    sgb::GpuBatchNormForwardTraining(bn, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                     nullptr, 0, nullptr);
    sgb::GpuBatchNormBackward(bn, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                              bn.workspace_bytes(), nullptr);
    sgb::GpuPoolingForward(mp, nullptr, nullptr, nullptr);
    sgb::GpuPoolingBackward(mp, nullptr, nullptr, nullptr, nullptr, nullptr);
    sgb::GpuPoolingForwardArgmax(mp, nullptr, nullptr, nullptr, nullptr);
    sgb::GpuPoolingBackwardArgmax(mp, nullptr, nullptr, nullptr, nullptr);
    sgb::GpuConvBackwardb(nullptr, nullptr, 1, 1, 1, 1, nullptr, 0, nullptr);
    sgb::NcclIdHolder id;
    sgb::Communicator c(0, 1, id, 1024);
    sgb::TensorRef t{nullptr, 0, false};
    c.synch(t, nullptr);
    c.fusedSynch({t}, nullptr, false);
    c.fusedSynch({t}, nullptr);
    c.synchHalf(t, nullptr);
    c.fusedSynchHalf({t}, nullptr);
    c.sparsification(t, nullptr, 0.01f, true, nullptr);
    c.fusedSparsification({t}, nullptr, 0.05f, false, nullptr);
    c.wait(nullptr);
    return c.global_rank + c.world_size + c.local_rank;
  }
  std::printf("%d\n", sgb_comm_unique_id_bytes());
  return 0;
}
''')
    exe = tmp_path / "use_communicator"
    libdir = os.path.dirname(lib_path)
    r = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(root, "include"),
                        str(src), "-o", str(exe), "-L", libdir, "-lsgb", "-Wl,-rpath," + libdir],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    # libsgb.so needs the NCCL that torch ships: make it findable for the child process
    import torch
    extra = [os.path.join(os.path.dirname(torch.__file__), "lib")]
    try:
        import nvidia.nccl
        extra.append(os.path.join(list(nvidia.nccl.__path__)[0], "lib"))
    except Exception:
        pass
    env = dict(os.environ, LD_LIBRARY_PATH=":".join(extra + [os.environ.get("LD_LIBRARY_PATH", "")]))
    out = subprocess.run([str(exe)], capture_output=True, text=True, env=env)
    assert out.returncode == 0, out.stderr
    assert int(out.stdout.strip()) == _lib.lib().sgb_comm_unique_id_bytes()
