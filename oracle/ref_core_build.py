"""Compiles apache/singa's own core library for its lang::Cpp (CPU) back end,
straight from the source tree, into ``oracle/_ref/libref_core.so``.

Sources, read where they lie (nothing is copied): ``src/core/tensor/tensor.cc``
(which pulls in ``tensor_math_cpp.h``, the CPU implementation of every tensor
operation), ``sparse_tensor.cc``, ``src/core/device/{device,cpp_cpu}.cc``,
``src/core/scheduler/scheduler.cc``, ``src/core/common/common.cc`` and
``src/utils/logging.cc``.  What the reference's CMake would generate or link
is replaced by three authored shims under ``oracle/ref_shims/``:

  singa/singa_config.h   CPU_ONLY + USE_CBLAS
  singa/proto/core.pb.h  the enums / messages of src/proto/core.proto (no protoc here)
  cblas.h + ref_cblas.c  the eight CBLAS routines the back end calls, OpenMP loops
                         (no CBLAS library here)

``ref_core_doors.cc`` adds extern "C" doors for the checker: the MLP training
step of benchmark configuration 1 on ``singa::Tensor`` objects, and single
operations for cross-checks.  TEST INFRASTRUCTURE ONLY: the library is the
CPU comparator / baseline; nothing under ``singa_b200/`` loads it.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("SINGA_REFERENCE", "/root/reference")
OUT = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "ref_shims")
LIB = os.path.join(OUT, "libref_core.so")

SOURCES = [
    "src/core/tensor/tensor.cc", "src/core/tensor/sparse_tensor.cc", "src/core/device/device.cc",
    "src/core/device/cpp_cpu.cc", "src/core/scheduler/scheduler.cc", "src/core/common/common.cc",
    "src/utils/logging.cc",
]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_ref_core(force=False):
    """Returns the library path, or None when the reference tree is absent."""
    srcs = [os.path.join(REFERENCE, s) for s in SOURCES]
    if not all(os.path.exists(s) for s in srcs):
        return LIB if os.path.exists(LIB) else None
    mine = [os.path.join(HERE, "ref_core_doors.cc"), os.path.join(SHIMS, "ref_cblas.c"),
            os.path.join(SHIMS, "cblas.h"), os.path.join(SHIMS, "singa", "proto", "core.pb.h"),
            os.path.join(SHIMS, "singa", "singa_config.h")]
    if not force and not _stale(LIB, srcs + mine):
        return LIB
    objdir = os.path.join(OUT, "core_obj")
    os.makedirs(objdir, exist_ok=True)
    inc = ["-I", SHIMS, "-I", os.path.join(REFERENCE, "include"),
           "-I", os.path.join(REFERENCE, "src", "core", "tensor")]
    # <cstring> / <cstdint> are forced in: two of the sources rely on older
    # standard headers pulling them in transitively.
    # AVX2 + FMA only (no -march=native): the library is built on one machine and
    # timed on another.
    cxx = ["g++", "-std=c++14", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-w", "-include", "cstring",
           "-include", "cstdint"] + inc
    objs = []
    procs = []
    for s in srcs + [mine[0]]:
        o = os.path.join(objdir, os.path.basename(s).rsplit(".", 1)[0] + ".o")
        objs.append(o)
        procs.append(subprocess.Popen(cxx + ["-c", s, "-o", o]))
    o = os.path.join(objdir, "ref_cblas.o")
    objs.append(o)
    procs.append(subprocess.Popen(["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-I", SHIMS, "-c", mine[1],
                                   "-o", o]))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("compiling the reference core failed")
    subprocess.check_call(["g++", "-shared", "-fopenmp", "-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    print(build_ref_core(force=True))
