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
    the compiled reference, tests/golden/make_golden.py), except the three
    Thrust helpers whose only caller - the communicator - is replaced."""
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
    missing = sorted(want - have)
    assert all(any(k in m for k in ("removezeroval", "removezeroidx", "sortbykey")) for m in missing), missing
    assert len(missing) == 3
    assert not (have - want), sorted(have - want)
    ctypes.CDLL(build.ADAPTER_LIB)       # resolves libsgb.so through its $ORIGIN runpath
