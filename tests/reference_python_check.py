"""numpy statement of the MLP steps that tests/reference_python_worker.py runs
through the reference's Python layer, and the comparison."""
import numpy as np


def numpy_steps(r, steps=3, lr=0.05, momentum=0.9, half=False):
    names = sorted(k[5:] for k in r.files if k.startswith("init:"))
    P = {n: r["init:" + n].astype(np.float32).copy() for n in names}
    W1 = next(n for n in names if "l1" in n and P[n].ndim == 2)
    b1 = next(n for n in names if "l1" in n and P[n].ndim == 1)
    W2 = next(n for n in names if "l2" in n and P[n].ndim == 2)
    b2 = next(n for n in names if "l2" in n and P[n].ndim == 1)
    M = {n: np.zeros_like(P[n]) for n in names}
    x, y = r["x"], r["y"]
    B = x.shape[0]
    losses = []
    for _ in range(steps):
        h = x @ P[W1] + P[b1]
        a = np.maximum(h, 0)
        z = a @ P[W2] + P[b2]
        z = z - z.max(1, keepdims=True)
        p = np.exp(z)
        p /= p.sum(1, keepdims=True)
        losses.append(float(-np.log(np.maximum(p[np.arange(B), y], np.finfo(np.float32).tiny)).sum() / B))
        dz = p.copy()
        dz[np.arange(B), y] -= 1
        dz /= B
        g = {W2: a.T @ dz, b2: dz.sum(0)}
        da = dz @ P[W2].T
        dh = np.where(h > 0, da, 0)
        g[W1], g[b1] = x.T @ dh, dh.sum(0)
        for n in names:
            gn = g[n].astype(np.float32)
            if half:
                gn = gn.astype(np.float16).astype(np.float32)
            M[n] = (momentum * M[n] + gn).astype(np.float32)
            P[n] = (P[n] - lr * M[n]).astype(np.float32)
    return losses, P


def check(r, rtol, half=False):
    losses, P = numpy_steps(r, half=half)
    got = r["losses"]
    assert got[-1] < got[0], "the loss does not go down: %s" % got
    np.testing.assert_allclose(got, losses, rtol=max(rtol, 1e-5))
    for n, want in P.items():
        g = r["final:" + n]
        scale = max(np.abs(want).max(), 1e-30)
        assert np.abs(g - want).max() <= rtol * scale, "%s: rel %.3e" % (n, np.abs(g - want).max() / scale)
