"""Compiles comparator objects straight from an apache/singa source tree.

Outputs go to ``oracle/_ref/`` only (git-ignored; they travel with a snapshot
of the repository like any other built library).  Nothing is copied from the
reference: nvcc reads ``src/core/tensor/math_kernel.cu`` where it lies.

``libref_cuda.so``   the reference's own CUDA launchers (math_kernel.cu,
                     unmodified, compiled for sm_100a) behind ``ref_shim.cu``.
                     Needs two things the reference's CMake would provide: a
                     ``singa/singa_config.h`` (generated here: USE_CUDA only)
                     and ``<thrust/count.h>``, which math_kernel.cu uses
                     without including (forced with -include).
``libref_cudnn.so``  the cuDNN calls the reference issues for BN / pooling
                     backward (``ref_cudnn.cu``, our harness; cuDNN is the
                     reference's third-party dependency, not vendored).

The rest of libsinga is not buildable here (needs cmake-generated protobuf
code, glog, cnmem and APIs removed from cuDNN 8 / CUDA 12).
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("SINGA_REFERENCE", "/root/reference")
OUT = os.path.join(HERE, "_ref")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
        "-shared", "-w"]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_ref(force=False):
    os.makedirs(os.path.join(OUT, "include", "singa"), exist_ok=True)
    cfg = os.path.join(OUT, "include", "singa", "singa_config.h")
    if not os.path.exists(cfg):
        with open(cfg, "w") as f:
            f.write("#ifndef SINGA_CONFIG_H_\n#define SINGA_CONFIG_H_\n#define USE_CUDA\n#endif\n")
    built = []
    kern = os.path.join(REFERENCE, "src", "core", "tensor", "math_kernel.cu")
    shim = os.path.join(HERE, "ref_shim.cu")
    lib = os.path.join(OUT, "libref_cuda.so")
    if os.path.exists(kern) and (force or _stale(lib, [kern, shim])):
        subprocess.check_call(["nvcc"] + ARCH + ["-I", os.path.join(OUT, "include"),
                                                 "-I", os.path.dirname(kern), "-include", "thrust/count.h",
                                                 kern, shim, "-o", lib])
    if os.path.exists(lib):
        built.append(lib)
    src = os.path.join(HERE, "ref_cudnn.cu")
    lib2 = os.path.join(OUT, "libref_cudnn.so")
    if force or _stale(lib2, [src]):
        subprocess.check_call(["nvcc"] + ARCH + [src, "-o", lib2, "-lcudnn"])
    built.append(lib2)
    return built


if __name__ == "__main__":
    for b in build_ref(force=True):
        print(b)
