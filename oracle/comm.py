"""numpy restatement of the communicator arithmetic, all ranks in one process.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Every function takes
the per-rank inputs as a list (index = rank) and returns what every rank
would hold after the collective.  Follows src/io/communicator.cc and
python/singa/opt.py of apache/singa as cited per function.

Parity status: the reference pins these paths only with constant inputs
(test/python/test_dist.py:37-121: grad=1, param=10 -> 10-0.1), which the
tests replay; ordering, ties, residuals and fp16 rounding are unpinned by the
reference and follow its source.
"""
import numpy as np

from . import cpu


# ----------------------------------------------------------------- bucketing
def plan_buckets(sizes, threshold=2097152):
    """Replays the bucket policy of DistOpt.backward_and_update
    (python/singa/opt.py:846-862) over gradient sizes given in the order the
    gradients are produced.  Returns a list of ("direct", [i]) and
    ("fused", [i, ...]) events in issue order."""
    events, glist, acc = [], [], 0
    for i, n in enumerate(sizes):
        if n > threshold:
            events.append(("direct", [i]))
        else:
            glist.append(i)
            acc += n
            if acc > threshold:
                events.append(("fused", glist))
                glist, acc = [], 0
    if glist:
        events.append(("fused", glist))
    return events


# ------------------------------------------------------------- dense all-reduce
def allreduce_sum(rank_tensors):
    """ncclAllReduce(sum) in fp32 (communicator.cc:141-145).  Summed in float64
    and rounded once: NCCL's order is unspecified, the tolerance is 1e-5."""
    s = np.zeros(rank_tensors[0].shape, np.float64)
    for t in rank_tensors:
        s += t.astype(np.float64)
    return s.astype(np.float32)


def allreduce_half(rank_tensors):
    """fp16 synchronisation (communicator.cc:330-467): each rank rounds its fp32
    gradient to half (round-to-nearest-even, math_kernel.cu:613-618), the halves
    are summed, the result is widened back to fp32.  No scaling before the sum.
    The sum of halves is formed in float32 and rounded to half once."""
    s = np.zeros(rank_tensors[0].shape, np.float32)
    for t in rank_tensors:
        s += t.astype(np.float32).astype(np.float16).astype(np.float32)
    return s.astype(np.float16).astype(np.float32)


def divide_by_world(t, world):
    """DistOpt.update: grad /= world_size (opt.py:738-746), which is a multiply
    by the fp32 reciprocal (src/core/tensor/tensor_math.h:149-153)."""
    return (t.astype(np.float32) * np.float32(1.0 / world)).astype(np.float32)


# ------------------------------------------------------------------ sparse sync
def topk_count(ratio, n):
    """nnzMax = (int)ceil(threshold * num) evaluated in fp32
    (communicator.cc:744: float * size_t -> float)."""
    return int(np.ceil(np.float32(ratio) * np.float32(n)))


def topk_keys(s, mode):
    """Sort key of the top-K selection.  "compat" is what the reference's
    comparator evaluates: both operands are truncated to int before |.| is
    taken (math_kernel.cu:715-721), so every |value| < 1 ties.  "magnitude" is
    the intended key |value|."""
    if mode == "compat":
        return np.abs(np.trunc(s.astype(np.float64))).astype(np.int64)
    if mode == "magnitude":
        return np.abs(s.astype(np.float32))
    raise ValueError(mode)


def topk_select(s, k, mode):
    """0-based indices of the k largest keys, ties broken by lower index,
    returned in ascending index order (the index SET is what parity checks)."""
    key = topk_keys(s, mode)
    if mode == "compat":
        order = np.argsort(-key, kind="stable")
    else:
        order = np.argsort(-key.astype(np.float64), kind="stable")
    return np.sort(order[:k]).astype(np.int64)


def _reduce_payloads(n, payloads):
    dense = np.zeros(n, np.float32)
    for idx, val in payloads:          # ascending rank order, communicator.cc:704
        cpu.scatter_add(dense, idx, val)
    return dense


def sparse_threshold_step(rank_grads, rank_accs, thr):
    """One valSparsAllReduce (communicator.cc:619-719) for all ranks.
    rank_accs is a list of residual arrays or None (corr=False).
    Returns (dense_sum, new_accs, payloads[(idx1, val)])."""
    payloads, new_accs = [], []
    for r, g in enumerate(rank_grads):
        acc = None if rank_accs is None else rank_accs[r]
        idx, val, acc2 = cpu.sparse_threshold(g, acc, thr)
        payloads.append((idx, val))
        new_accs.append(acc2)
    dense = _reduce_payloads(rank_grads[0].size, payloads)
    return dense, (None if rank_accs is None else new_accs), payloads


def sparse_threshold_bounded_step(rank_grads, rank_accs, thr, capacity):
    """The capacity-bounded threshold exchange (an addition of this library, no
    counterpart in the reference): the selection rule of valSparsAllReduce
    (communicator.cc:619-680), but every rank sends only its first `capacity`
    selected entries in index order; the others stay in the residual (or are
    lost when there is none).  Returns (dense_sum, new_accs, held_back per rank)."""
    payloads, new_accs, held = [], [], []
    for r, g in enumerate(rank_grads):
        acc = None if rank_accs is None else rank_accs[r]
        idx, val, acc2 = cpu.sparse_threshold(g, acc, thr)
        keep = min(len(idx), int(capacity))
        if acc2 is not None and keep < len(idx):
            acc2[idx[keep:] - 1] = val[keep:]          # not sent: back into the residual, bit for bit
        payloads.append((idx[:keep], val[:keep]))
        new_accs.append(acc2)
        held.append(len(idx) - keep)
    dense = _reduce_payloads(rank_grads[0].size, payloads)
    return dense, (None if rank_accs is None else new_accs), held


def sparse_topk_step(rank_grads, rank_accs, ratio, mode="magnitude"):
    """One topKSparsAllReduce (communicator.cc:721-807) for all ranks:
    s = g + acc; the K = ceil(ratio*n) entries with the largest key are sent;
    acc' = s with the sent entries zeroed."""
    n = rank_grads[0].size
    k = topk_count(ratio, n)
    payloads, new_accs = [], []
    for r, g in enumerate(rank_grads):
        g = np.asarray(g, np.float32).ravel()
        s = g if rank_accs is None else (g + rank_accs[r].ravel()).astype(np.float32)
        sel = topk_select(s, k, mode)
        payloads.append(((sel + 1).astype(np.int32), s[sel].copy()))
        if rank_accs is not None:
            a = s.copy()
            a[sel] = 0.0
            new_accs.append(a)
    dense = _reduce_payloads(n, payloads)
    return dense, (None if rank_accs is None else new_accs), payloads
