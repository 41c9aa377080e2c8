"""nvcc recipe for the C-ABI library ``libsgb.so`` (sm_100a only).

The library is built in-tree, next to the sources, so that it travels with a
snapshot of the repository.  ``python -m singa_b200.build`` rebuilds it.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libsgb.so")
ADAPTER_SRC = os.path.join(HERE, "adapter", "singa_cuda_launchers.cu")
ADAPTER_LIB = os.path.join(HERE, "libsgb_singa.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
    "-std=c++17", "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC,
]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "sgb.h"))
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, verbose):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    path = os.path.join(CSRC, src)
    if _stale(obj, [path] + _headers()):
        cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stderr))
        if verbose:
            sys.stderr.write(r.stderr)
    return obj


def build(verbose=False, force=False):
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in os.listdir(OBJ):
            os.remove(os.path.join(OBJ, f))
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), sources()))
    if _stale(LIB, objs):
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lnccl", "-lcudart"]
        subprocess.check_call(cmd)
    build_adapter()
    return LIB


def build_adapter():
    """libsgb_singa.so: the `singa::cuda::*` launchers (C++ linkage, the
    reference's signatures) forwarding to libsgb.so, found through $ORIGIN."""
    if _stale(ADAPTER_LIB, [ADAPTER_SRC, LIB, os.path.join(INCLUDE, "sgb.h")]):
        cmd = ["nvcc"] + NVCC_FLAGS + ["-shared", ADAPTER_SRC, "-o", ADAPTER_LIB, "-L", HERE, "-lsgb",
                                       "-Xlinker", "-rpath=$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for the launcher adapter:\n%s" % r.stderr)
    return ADAPTER_LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
