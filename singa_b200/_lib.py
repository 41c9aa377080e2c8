"""ctypes binding of ``libsgb.so`` - the only way the package reaches the GPU.

Prototypes are derived from ``include/sgb.h`` so the header stays the single
source of truth.  There is no CPU fallback: if the library is missing or a
call returns a non-zero status, an exception is raised.
"""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(HERE), "include", "sgb.h")
LIB_PATH = os.path.join(HERE, "libsgb.so")


class SgbError(RuntimeError):
    def __init__(self, fn, status, text):
        super().__init__("%s failed: status %d (%s)" % (fn, status, text))
        self.status = status


_SCALARS = {
    "int": C.c_int, "int32_t": C.c_int32, "unsigned": C.c_uint, "size_t": C.c_size_t,
    "float": C.c_float, "double": C.c_double, "uint64_t": C.c_uint64,
    "int64_t": C.c_int64, "uint32_t": C.c_uint32,
}


def declarations(header=HEADER):
    """[(name, restype, [argtype, ...])] for every function declared in sgb.h."""
    with open(header) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"enum\s+\w+\s*\{[^}]*\}\s*;", " ", text, flags=re.S)
    out = []
    for m in re.finditer(r"([\w\s\*]+?)\b(sgb_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if "typedef" in ret:
            continue
        restype = C.c_char_p if "char" in ret else (C.c_void_p if "*" in ret else
                                                    (C.c_size_t if "size_t" in ret else C.c_int))
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    argtypes.append(C.c_void_p)
                else:
                    toks = [t for t in a.split() if t not in ("const", "unsigned")]
                    ty = "unsigned" if a.startswith("unsigned") and len(toks) == 1 else toks[0]
                    argtypes.append(_SCALARS[ty])
        out.append((name, restype, argtypes))
    return out


_lib = None


def lib():
    """Loads libsgb.so (once) and installs the prototypes."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libsgb.so is not built (%s). Run `python -m singa_b200.build`; "
                "there is no CPU fallback." % LIB_PATH)
        # libsgb.so needs libnccl.so.2.  torch ships its own (newer) NCCL under the
        # same soname and must find THAT one already loaded, otherwise
        # libtorch_cuda fails to resolve its symbols: import torch first, then
        # our library binds to the copy torch loaded.
        import torch  # noqa: F401
        handle = C.CDLL(LIB_PATH)
        for name, restype, argtypes in declarations():
            fn = getattr(handle, name)   # AttributeError if the symbol is missing
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def call(name, *args):
    """Calls an int-returning entry point and raises SgbError on failure."""
    handle = lib()
    status = getattr(handle, name)(*args)
    if status != 0:
        text = handle.sgb_status_string(status).decode()
        if status == -3:
            text += " cudaError=%d" % handle.sgb_last_cuda_error()
        raise SgbError(name, status, text)
    return status
