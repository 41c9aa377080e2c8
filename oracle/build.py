"""Build recipes for the checker libraries.

``build_oracle()`` compiles ``oracle.c`` into ``oracle/liboracle.so`` with gcc.
``build_ref()`` (see ``oracle/ref_build.py``) compiles objects straight from an
apache/singa source tree when one is present; its outputs go to
``oracle/_ref/`` only.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "oracle.c")
    if force or _stale(LIB, [src]):
        cmd = ["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-std=c11",
               "-ffp-contract=off", "-o", LIB, src, "-lm"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build_oracle(force=True))
