"""Builds `singa_wrap` - the extension module apache/singa's Python layer
imports - with pybind11 (SWIG is not available), and assembles an importable
`singa` package around it from the reference's UNMODIFIED python/singa/*.py.

    python -m singa_b200.adapter.build_singa_wrap [cpp|sgb ...]

variant "cpp": the reference's own lang::Cpp core (oracle/_ref/libref_core.so);
               runs without a GPU.
variant "sgb": the reference's Tensor / Device sources with this repository's
               CUDA back end, operation adapters and communicator adapter
               (oracle/_ref/libsgb_singa_cuda.so).

Output: baseline/_ref/singa_<variant>/singa/ (git-ignored: it contains the
reference's Python files, copied, and objects compiled from its sources).  Put
baseline/_ref/singa_<variant> on sys.path and `import singa`.
"""
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE = os.environ.get("SINGA_REFERENCE", "/root/reference")
OUT = os.path.join(ROOT, "baseline", "_ref")
SOURCES = ["singa_wrap_pybind.cc", "singa_wrap_pybind_math.cc", "singa_wrap_pybind_ops.cc"]


def package_dir(variant):
    return os.path.join(OUT, "singa_" + variant, "singa")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(variant, force=False):
    """Returns the directory to put on sys.path, or None when the reference
    tree is absent and nothing was prebuilt."""
    sys.path.insert(0, ROOT)
    pkg = package_dir(variant)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    module = os.path.join(pkg, "singa_wrap" + ext)
    if not os.path.isdir(os.path.join(REFERENCE, "python", "singa")):
        return os.path.dirname(pkg) if os.path.exists(module) else None
    import pybind11
    from oracle import ref_core_build, ref_cuda_build
    if variant == "cpp":
        core = ref_core_build.build_ref_core()
        shims = [os.path.join(ROOT, "oracle", "ref_shims")]
        extra_inc = []
    else:
        core = ref_cuda_build.build_variant("sgb")
        shims = [HERE, os.path.join(ROOT, "oracle", "ref_shims_cuda"), os.path.join(ROOT, "oracle", "ref_shims")]
        extra_inc = ["-I", "/usr/local/cuda/include", "-I", os.path.join(ROOT, "include")]
    os.makedirs(pkg, exist_ok=True)
    srcs = [os.path.join(HERE, s) for s in SOURCES]
    if force or _stale(module, srcs + [core]):
        cmd = ["g++", "-std=c++14", "-O2", "-shared", "-fPIC", "-w", "-fvisibility=hidden", "-include", "cstring",
               "-include", "cstdint"]
        for s in shims:
            cmd += ["-I", s]
        cmd += ["-I", os.path.join(REFERENCE, "include"), "-I", os.path.join(REFERENCE, "src"),
                "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]] + extra_inc
        cmd += srcs + ["-o", module, core, "-Wl,-rpath," + os.path.dirname(core),
                       "-Wl,-rpath,$ORIGIN/../../../../oracle/_ref"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("building singa_wrap (%s) failed:\n%s" % (variant, r.stderr[-6000:]))
    # the reference's Python layer, file by file, unmodified
    src_pkg = os.path.join(REFERENCE, "python", "singa")
    for name in os.listdir(src_pkg):
        if name.endswith(".py"):
            dst = os.path.join(pkg, name)
            if _stale(dst, [os.path.join(src_pkg, name)]):
                shutil.copyfile(os.path.join(src_pkg, name), dst)
    return os.path.dirname(pkg)


if __name__ == "__main__":
    for v in (sys.argv[1:] or ["cpp"]):
        print(build(v, force=True))
