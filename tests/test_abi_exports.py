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
    for code in range(-8, 0):
        assert lib.sgb_status_string(code) != b"unknown status"


def test_argument_validation_needs_no_gpu():
    # NULL pointers and bad enums are rejected on the host before any launch.
    lib = _lib.lib()
    assert lib.sgb_relu_backward_f32(None, None, None, 0, None) == 0      # n == 0 is a no-op
    assert lib.sgb_relu_backward_f32(None, None, None, 16, None) == -1    # SGB_ERR_NULL
    assert lib.sgb_binary_f32(99, 1, 1, 1, 0, None) in (0, -6)
