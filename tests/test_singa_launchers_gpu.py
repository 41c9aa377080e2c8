"""Drop-in check at the C++ symbol level: every `singa::cuda::*` launcher of
libsgb_singa.so is called through its mangled name with the same device
buffers as the launcher of the same name in the reference's own compiled
math_kernel.cu (oracle/_ref/libref_cuda.so), and the outputs are compared bit
for bit.  The argument pattern of each launcher is read off its mangled
signature, so a launcher added on either side is picked up automatically."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
OURS = os.path.join(ROOT, "singa_b200", "libsgb_singa.so")
SYMS = os.path.join(ROOT, "tests", "golden", "singa_cuda_launcher_symbols.txt")
N = 100003

# launchers whose last bits may legitimately differ from the reference's
# (different but equally valid evaluation of a transcendental): name -> max ulp
ULP = {}


class Half(C.Structure):          # a __half passed by value
    _fields_ = [("x", C.c_uint16)]


def split(sym):
    m = re.match(r"_ZN5singa4cuda(\d+)", sym)
    k = int(m.group(1))
    start = m.end()
    return sym[start:start + k], sym[start + k + 1:]     # name, parameter encoding


def symbols():
    with open(SYMS) as f:
        return [s for s in f.read().split() if not any(k in s for k in ("removezero", "sortbykey"))]


@pytest.fixture(scope="module")
def libs():
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libref_cuda.so not built")
    from singa_b200 import _lib
    _lib.lib()
    return C.CDLL(REF), C.CDLL(OURS)


def domain(name, rng, n):
    if name in ("log", "sqrt", "acosh", "pow"):
        return rng.uniform(1.0, 3.0, n).astype(np.float32)
    if name in ("acos", "asin", "atanh"):
        return rng.uniform(-0.95, 0.95, n).astype(np.float32)
    x = rng.standard_normal(n).astype(np.float32) * 2
    x[::17] = 0.0
    x[5::29] = np.round(x[5::29])
    return x


def p(t):
    return C.c_void_p(t.data_ptr())


def run_case(name, enc, fn, rng):
    """Builds inputs for the launcher's signature, calls it, returns outputs."""
    f32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    f16 = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda().half()
    a, b = domain(name, rng, N), domain(name, rng, N)
    b[::13] = a[::13]                                   # ties for the comparisons
    n = C.c_size_t(N)
    s = None
    if enc == "mfPfP11CUstream_st":                      # set
        out = torch.empty(N, device="cuda")
        fn(n, C.c_float(1.25), p(out), s)
    elif enc == "mPKfPfP11CUstream_st":
        out = torch.empty(N, device="cuda")
        fn(n, p(f32(a)), p(out), s)
    elif enc == "mPKfS2_PfP11CUstream_st":
        out = torch.empty(N, device="cuda")
        fn(n, p(f32(a)), p(f32(b)), p(out), s)
    elif enc == "mPKffPfP11CUstream_st":
        out = torch.empty(N, device="cuda")
        fn(n, p(f32(a)), C.c_float(a[13] if name in ("eq", "ge", "le") else 0.75), p(out), s)
    elif enc == "mfPKfPfP11CUstream_st":
        out = torch.empty(N, device="cuda")
        fn(n, C.c_float(0.75), p(f32(a)), p(out), s)
    elif enc == "mffPKfPfP11CUstream_st":
        out = torch.empty(N, device="cuda")
        fn(n, C.c_float(-0.5), C.c_float(0.8), p(f32(a)), p(out), s)
    elif enc == "mPK6__halfPS1_P11CUstream_st":
        out = torch.empty(N, device="cuda", dtype=torch.float16)
        fn(n, p(f16(a)), p(out), s)
    elif enc == "mPK6__halfS3_PS1_P11CUstream_st":
        out = torch.empty(N, device="cuda", dtype=torch.float16)
        fn(n, p(f16(a)), p(f16(b)), p(out), s)
    elif enc == "mPK6__halfS1_PS1_P11CUstream_st":
        out = torch.empty(N, device="cuda", dtype=torch.float16)
        fn(n, p(f16(a)), Half(int(np.float16(0.75).view(np.uint16))), p(out), s)
    elif enc == "mPKfPiP11CUstream_st":
        out = torch.empty(N, device="cuda", dtype=torch.int32)
        fn(n, p(f32(a * 100)), p(out), s)
    elif enc == "mPKiPfP11CUstream_st":
        out = torch.empty(N, device="cuda")
        fn(n, p(torch.from_numpy(rng.integers(-10 ** 6, 10 ** 6, N).astype(np.int32)).cuda()), p(out), s)
    elif enc == "mPKfP6__halfP11CUstream_st":
        out = torch.empty(N, device="cuda", dtype=torch.float16)
        fn(n, p(f32(a * 100)), p(out), s)
    elif enc == "mPK6__halfPfP11CUstream_st":
        out = torch.empty(N, device="cuda")
        fn(n, p(f16(a)), p(out), s)
    elif enc == "mPiP11CUstream_st":
        out = torch.empty(N, device="cuda", dtype=torch.int32)
        fn(n, p(out), s)
    elif enc == "mmPKfPfP11CUstream_st":                 # RowMax
        rows, cols = 257, 389
        out = torch.empty(rows, device="cuda")
        fn(C.c_size_t(rows), C.c_size_t(cols), p(f32(a[:rows * cols])), p(out), s)
    elif enc in ("mmPKfPKiS4_PfP11CUstream_st", "mmPK6__halfPKiS5_PS1_P11CUstream_st"):
        half = "__half" in enc                            # transposed + broadcast view of a (5, 1, 7) storage
        shape, stride = (7, 3, 5), (1, 0, 7)
        src = (f16 if half else f32)(a[:35])
        out = torch.empty(105, device="cuda", dtype=torch.float16 if half else torch.float32)
        sh = torch.tensor(shape, dtype=torch.int32, device="cuda")
        st = torch.tensor(stride, dtype=torch.int32, device="cuda")
        fn(C.c_size_t(105), C.c_size_t(3), p(src), p(sh), p(st), p(out), s)
    elif enc in ("bmmPKfPKiPfP11CUstream_st", "bmmPK6__halfPKiPS1_P11CUstream_st"):
        half = "__half" in enc
        batch, dim = 61, 37
        logits = rng.standard_normal((batch, dim)).astype(np.float32)
        prob = np.exp(logits) / np.exp(logits).sum(1, keepdims=True)
        prob[3, 5] = 0.0
        outs = []
        for int_target in (True, False):
            t = rng.integers(0, dim, batch) if int_target else rng.integers(0, 4, (batch, dim))
            if not int_target:
                t[:, 0] += 1
            t = torch.from_numpy(t.astype(np.int32)).cuda()
            pd = (f16 if half else f32)(prob)
            if name == "ComputeCrossEntropy":
                out = torch.zeros(batch, device="cuda", dtype=pd.dtype)
            else:
                out = pd.clone()                          # the caller hands over a clone of p
            fn(C.c_bool(int_target), C.c_size_t(batch), C.c_size_t(dim), p(pd), p(t), p(out), s)
            outs.append(out)
        torch.cuda.synchronize()
        return outs
    else:
        raise AssertionError("unhandled signature %s %s" % (name, enc))
    torch.cuda.synchronize()
    return [out]


def as_int(t):
    return t.view(torch.int32 if t.element_size() == 4 else torch.int16)


@pytest.mark.parametrize("sym", symbols())
def test_launcher_matches_reference_launcher(libs, sym):
    ref, ours = libs
    name, enc = split(sym)
    outs = []
    for lib in (ref, ours):
        fn = getattr(lib, sym)
        fn.restype = None
        outs.append(run_case(name, enc, fn, np.random.default_rng(len(sym))))
    for r, o in zip(*outs):
        if name in ULP:
            d = (as_int(r).long() - as_int(o).long()).abs().max().item()
            assert d <= ULP[name], "%s: %d ulp" % (name, d)
        else:
            same = as_int(r) == as_int(o)
            both_nan = torch.isnan(r.float()) & torch.isnan(o.float())
            bad = ~(same | both_nan)
            assert not bad.any(), "%s(%s): %d of %d elements differ, first at %d: %r vs %r" % (
                name, enc, int(bad.sum()), bad.numel(), int(bad.flatten().nonzero()[0]),
                r.flatten()[bad.flatten()][0].item(), o.flatten()[bad.flatten()][0].item())


def _by_name(lib, needle):
    with open(SYMS) as f:
        sym = next(s for s in f.read().split() if needle in s)
    return getattr(lib, sym)


def test_compaction_and_sort_helpers_match_the_reference(libs):
    """The three helpers the reference builds on Thrust, through their mangled
    names on both libraries: removezeroval (same compacted prefix), sortbykey
    (same pairs in the same order: the comparator sees integer-truncated
    magnitudes, ties keep their original order) and removezeroidx (same
    compacted prefix; the count is the number of non-zero entries, which is
    what the reference's caller needs - its own count reads the unspecified
    tail that thrust::remove leaves behind)."""
    ref, ours = libs
    rng = np.random.default_rng(8)
    n = 300007
    v = (rng.standard_normal(n) * 3).astype(np.float32)
    v[rng.random(n) < 0.6] = 0.0
    v[7] = -0.0
    kept = v[v != 0]
    outs = []
    for lib in (ref, ours):
        t = torch.from_numpy(v.copy()).cuda()
        _by_name(lib, "removezeroval")(C.c_size_t(n), C.c_void_p(t.data_ptr()), None)
        torch.cuda.synchronize()
        outs.append(t.cpu().numpy()[:kept.size])
    assert np.array_equal(outs[0], kept) and np.array_equal(outs[1], kept)

    idx = np.where(v != 0, np.arange(1, n + 1), 0).astype(np.int32)
    t = torch.from_numpy(idx.copy()).cuda()
    count = C.c_int(-1)
    _by_name(ours, "removezeroidx")(C.c_size_t(n), C.c_void_p(t.data_ptr()), None, C.byref(count))
    torch.cuda.synchronize()
    assert count.value == kept.size
    assert np.array_equal(t.cpu().numpy()[:kept.size], idx[idx != 0])

    for scale in (3.0, 1e-3):                      # distinct integer keys / everything ties at 0
        key = (rng.standard_normal(n) * scale).astype(np.float32)
        val = np.arange(1, n + 1, dtype=np.int32)
        res = []
        for lib in (ref, ours):
            k, w = torch.from_numpy(key.copy()).cuda(), torch.from_numpy(val.copy()).cuda()
            _by_name(lib, "sortbykey")(C.c_size_t(n), C.c_void_p(k.data_ptr()), C.c_void_p(w.data_ptr()), None)
            torch.cuda.synchronize()
            res.append((k.cpu().numpy(), w.cpu().numpy()))
        assert np.array_equal(res[0][1], res[1][1]), "index order differs at scale %g" % scale
        assert np.array_equal(res[0][0], res[1][0])
        mags = np.abs(res[1][0].astype(np.int32))
        assert (np.diff(mags) <= 0).all()
