"""Builds apache/singa's core library for CUDA, straight from its source tree,
in two variants that share everything except the CUDA back end:

``oracle/_ref/libref_singa_cuda.so``  (variant "reference")
    the reference's own CUDA path, unmodified: tensor.cc with its
    tensor_math_cuda.h, math_kernel.cu, the cuDNN batch-norm / pooling
    operations (src/model/operation/{batchnorm,pooling}.cc) and
    src/io/communicator.cc.  This is the GPU comparator.

``oracle/_ref/libsgb_singa_cuda.so``   (variant "sgb")
    the same Tensor / Device / Scheduler sources with THIS repository's
    replacement back end plugged in at the reference's build-time plug-in
    points: ``singa_b200/adapter/tensor_math_cuda.h`` instead of the
    reference's header (tensor.cc includes the three back-end headers once,
    src/core/tensor/tensor.cc:22-25), ``libsgb_singa.so`` instead of
    math_kernel.cu, ``singa_b200/adapter/operations.cc`` instead of the Gpu*
    backward functions and ``singa_b200/adapter/communicator.cc`` instead of
    src/io/communicator.cc.

Both carry the same extern "C" doors (``ref_cuda_doors.cc``), written against
the reference's public C++ interface only.  What the reference's build would
generate or link and is absent here is replaced by authored shims under
``oracle/ref_shims*/``: singa_config.h, core.pb.h (no protoc), cblas.h (no
CBLAS), cnmem.h (cnmem is an external dependency), mpi.h (no MPI; only the
NCCL-id constructor is used) and cusparseSaxpyi (removed in CUDA 12).
Nothing is copied from the reference; outputs go to ``oracle/_ref/`` only.
src/model/operation/convolution.cc is not built: it uses cuDNN enums that
were removed in cuDNN 8.
"""
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REFERENCE = os.environ.get("SINGA_REFERENCE", "/root/reference")
OUT = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "ref_shims")
SHIMS_CUDA = os.path.join(HERE, "ref_shims_cuda")
ADAPTER = os.path.join(ROOT, "singa_b200", "adapter")
PKG = os.path.join(ROOT, "singa_b200")

CORE = [
    "src/core/tensor/sparse_tensor.cc", "src/core/device/device.cc", "src/core/device/cpp_cpu.cc",
    "src/core/device/cuda_gpu.cc", "src/core/device/platform.cc", "src/core/memory/memory.cc",
    "src/core/scheduler/scheduler.cc", "src/core/common/common.cc", "src/utils/logging.cc",
]
LIBS = {"reference": os.path.join(OUT, "libref_singa_cuda.so"), "sgb": os.path.join(OUT, "libsgb_singa_cuda.so")}


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def _includes():
    return ["-I", SHIMS_CUDA, "-I", SHIMS, "-I", os.path.join(REFERENCE, "include"),
            "-I", os.path.join(REFERENCE, "src"), "-I", os.path.join(REFERENCE, "src", "core", "tensor"),
            "-I", "/usr/local/cuda/include", "-I", os.path.join(ROOT, "include")]


def _cxx(src, obj, extra=()):
    cmd = ["g++", "-std=c++14", "-O2", "-fopenmp", "-fPIC", "-w", "-include", "cstring", "-include", "cstdint",
           "-include", os.path.join(SHIMS_CUDA, "saxpyi_compat.h")] + list(extra) + _includes() + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed for %s:\n%s" % (src, r.stderr[-4000:]))
    return obj


def _nvcc(src, obj, extra=()):
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-w",
           "-I", SHIMS_CUDA] + _includes()[2:] + list(extra) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stderr[-4000:]))
    return obj


def build_variant(variant, force=False):
    """Returns the library path, or None when neither the reference tree nor a
    prebuilt library is present."""
    lib = LIBS[variant]
    ref = lambda p: os.path.join(REFERENCE, p)
    if not os.path.exists(ref("src/core/tensor/tensor.cc")):
        return lib if os.path.exists(lib) else None
    doors = os.path.join(HERE, "ref_cuda_doors.cc")
    shim_files = [os.path.join(SHIMS_CUDA, f) for f in ("cnmem.h", "mpi.h", "saxpyi_compat.h", "saxpyi_compat.cu",
                                                        os.path.join("singa", "singa_config.h"))]
    mine = []
    if variant == "sgb":
        mine = [os.path.join(ADAPTER, f) for f in ("tensor_math_cuda.h", "tensor_with_sgb_backend.cc",
                                                   "operations.cc", "communicator.cc",
                                                   os.path.join("singa", "io", "communicator.h"))]
        mine += [os.path.join(PKG, "libsgb.so"), os.path.join(PKG, "libsgb_singa.so")]
    deps = [ref(s) for s in CORE] + [ref("src/core/tensor/tensor.cc"), doors] + shim_files + mine
    if not force and not _stale(lib, deps):
        return lib
    objdir = os.path.join(OUT, "cuda_obj_" + variant)
    os.makedirs(objdir, exist_ok=True)
    jobs = []

    def obj(name):
        return os.path.join(objdir, name + ".o")

    for s in CORE:
        jobs.append((_cxx, ref(s), obj(os.path.basename(s)[:-3]), ()))
    jobs.append((_cxx, ref("src/model/operation/pooling.cc"), obj("pooling"),
                 ("-DGpuPoolingBackward=GpuPoolingBackward_reference",) if variant == "sgb" else ()))
    jobs.append((_cxx, ref("src/model/operation/batchnorm.cc"), obj("batchnorm"),
                 ("-DGpuBatchNormBackward=GpuBatchNormBackward_reference",) if variant == "sgb" else ()))
    jobs.append((_cxx, doors, obj("doors"),
                 ("-I", ADAPTER, "-DSGB_VARIANT") if variant == "sgb" else ()))
    if variant == "reference":
        jobs.append((_cxx, ref("src/core/tensor/tensor.cc"), obj("tensor"), ()))
        jobs.append((_cxx, ref("src/io/communicator.cc"), obj("communicator"), ()))
        jobs.append((_nvcc, ref("src/core/tensor/math_kernel.cu"), obj("math_kernel"), ("-include", "thrust/count.h")))
        jobs.append((_nvcc, os.path.join(SHIMS_CUDA, "saxpyi_compat.cu"), obj("saxpyi"), ()))
    else:
        jobs.append((_cxx, os.path.join(ADAPTER, "tensor_with_sgb_backend.cc"), obj("tensor"), ("-I", ADAPTER)))
        jobs.append((_cxx, os.path.join(ADAPTER, "operations.cc"), obj("operations"), ("-I", ADAPTER)))
        jobs.append((_cxx, os.path.join(ADAPTER, "communicator.cc"), obj("communicator"), ("-I", ADAPTER)))
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda j: j[0](j[1], j[2], j[3]), jobs))
    objs.append(_cblas(obj("ref_cblas")))
    link = ["g++", "-shared", "-fopenmp", "-o", lib] + objs + ["-L/usr/local/cuda/lib64", "-lcudart", "-lcublas",
                                                             "-lcurand", "-lcudnn", "-lcusparse", "-lnccl"]
    if variant == "sgb":
        link += ["-L", PKG, "-lsgb_singa", "-lsgb", "-Wl,-rpath," + PKG, "-Wl,-rpath,$ORIGIN/../../singa_b200"]
    subprocess.check_call(link)
    return lib


GTEST_SOURCES = ["test/gtest/gtest-all.cc", "test/gtest/gtest_main.cc", "test/singa/test_tensor_math.cc",
                 "test/singa/test_tensor.cc", "test/singa/test_cross_entropy.cc",
                 "src/model/loss/softmax_cross_entropy.cc"]


def gtest_binary(variant):
    return os.path.join(OUT, "singa_gtest_" + variant)


def build_gtests(variant, force=False):
    """The reference's OWN unit tests - test/singa/test_tensor_math.cc,
    test_tensor.cc and test_cross_entropy.cc (with the loss layer it drives,
    src/model/loss/softmax_cross_entropy.cc) and its vendored gtest - compiled
    unmodified and linked against one of the two core builds.  Returns the binary's path (None when
    neither the reference tree nor a prebuilt binary is present)."""
    lib = build_variant(variant)
    exe = gtest_binary(variant)
    ref = lambda p: os.path.join(REFERENCE, p)
    if lib is None or not os.path.exists(ref(GTEST_SOURCES[0])):
        return exe if os.path.exists(exe) else None
    if not force and not _stale(exe, [lib] + [ref(g) for g in GTEST_SOURCES]):
        return exe
    objdir = os.path.join(OUT, "gtest_obj_" + variant)
    os.makedirs(objdir, exist_ok=True)
    extra = ("-I", ref("test"))
    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(lambda g: _cxx(ref(g), os.path.join(objdir, os.path.basename(g)[:-3] + ".o"), extra),
                           GTEST_SOURCES))
    subprocess.check_call(["g++", "-o", exe] + objs + [lib, "-lpthread", "-L/usr/local/cuda/lib64", "-lcudart",
                           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../singa_b200", "-Wl,-rpath," + OUT,
                           "-Wl,-rpath," + PKG])
    return exe


def _cblas(obj):
    subprocess.check_call(["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-I", SHIMS, "-c",
                           os.path.join(SHIMS, "ref_cblas.c"), "-o", obj])
    return obj


if __name__ == "__main__":
    import sys
    for v in (sys.argv[1:] or ["reference"]):
        print(build_variant(v, force=True))
        print(build_gtests(v, force=True))
