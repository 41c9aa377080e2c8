"""``NcclIdHolder`` and ``Communicator`` with the reference's SWIG-level API
(src/api/dist_communicator.i:33-60) on top of the C-ABI communicator.

One process per GPU.  The unique id is created by one rank and shipped to the
others by the caller (``torch.distributed`` store / broadcast, a pipe, ...), as
``NcclIdHolder`` is in the reference's multiprocessing examples.
"""
import ctypes as C

import torch

from . import _lib


class NcclIdHolder(object):
    """Holds an ncclUniqueId (communicator.cc:49-51) as bytes."""

    def __init__(self, id_bytes=None):
        if id_bytes is None:
            n = _lib.lib().sgb_comm_unique_id_bytes()
            buf = C.create_string_buffer(n)
            _lib.call("sgb_comm_get_unique_id", C.cast(buf, C.c_void_p))
            id_bytes = buf.raw
        self.id = bytes(id_bytes)


def _table(tensors):
    n = len(tensors)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in tensors])
    sizes = (C.c_size_t * n)(*[t.numel() for t in tensors])
    return ptrs, sizes, n


def _stream():
    return torch.cuda.current_stream().cuda_stream


class Communicator(object):
    """Mirror of ``singa::Communicator`` (include/singa/io/communicator.h:76-95).

    Public fields ``global_rank``, ``world_size``, ``local_rank`` as in the
    reference.  All methods enqueue work and return; ``wait()`` makes the
    current (compute) stream wait for the communicator's side streams.
    """

    def __init__(self, local_rank, world_size, holder, buffSize=4194304, min_ctas=0, max_ctas=0):
        if not torch.cuda.is_available():
            raise RuntimeError("singa_b200.Communicator needs a CUDA device; there is no CPU path")
        self.local_rank = int(local_rank)
        self.global_rank = int(local_rank)
        self.world_size = int(world_size)
        torch.cuda.set_device(self.local_rank)
        torch.cuda.current_stream().synchronize()   # context exists before NCCL init
        handle = C.c_void_p()
        idbuf = C.create_string_buffer(holder.id, len(holder.id))
        self._h = None
        try:
            _lib.call("sgb_comm_create_ex", C.byref(handle), self.global_rank, self.world_size,
                      C.cast(idbuf, C.c_void_p), int(buffSize), int(min_ctas), int(max_ctas))
        except _lib.SgbError:
            if handle:
                _lib.lib().sgb_comm_destroy(handle)
            raise
        self._h = handle

    def close(self):
        if self._h is not None:
            _lib.lib().sgb_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_topk_mode(self, mode):
        """"compat" (default): the reference comparator's key; "magnitude": |g|."""
        _lib.call("sgb_comm_set_topk_mode", self._h, {"magnitude": 0, "compat": 1}[mode])

    def register(self, t):
        """Registers a tensor that is reduced in place (a gradient arena) with NCCL."""
        _lib.call("sgb_comm_register", self._h, t.data_ptr(), t.numel() * t.element_size())

    # -- per-phase device timing (the reference's per-operation time profiling)
    def profile_begin(self):
        _lib.call("sgb_comm_profile_begin", self._h, _stream())

    def profile_mark(self, name):
        _lib.call("sgb_comm_profile_mark", self._h, name.encode(), _stream())

    def profile_end(self, capacity=4096):
        """[(phase name, start ms, end ms)] since profile_begin, in issue order."""
        stride = 64
        names = C.create_string_buffer(stride * capacity)
        t0, t1 = (C.c_float * capacity)(), (C.c_float * capacity)()
        count = C.c_size_t()
        _lib.call("sgb_comm_profile_end", self._h, C.cast(names, C.c_void_p), stride, t0, t1, capacity,
                  C.byref(count))
        n = min(count.value, capacity)
        return [(names.raw[i * stride:(i + 1) * stride].split(b"\0", 1)[0].decode(), float(t0[i]), float(t1[i]))
                for i in range(n)]

    # -- reference API -------------------------------------------------------
    def synch(self, t):
        _lib.call("sgb_comm_synch", self._h, t.data_ptr(), t.numel(),
                  int(t.dtype == torch.float16), _stream())

    def fusedSynch(self, ts, send=True):
        ptrs, sizes, n = _table(ts)
        _lib.call("sgb_comm_fused_synch", self._h, ptrs, sizes, n,
                  int(ts[0].dtype == torch.float16), int(send), _stream())

    def synchHalf(self, t):
        assert t.dtype == torch.float32, \
            "only available for 32-bit tensors, which are converted to 16 bits before transmit"
        _lib.call("sgb_comm_synch_half", self._h, t.data_ptr(), t.numel(), _stream())

    def fusedSynchHalf(self, ts, send=True):
        assert ts[0].dtype == torch.float32
        ptrs, sizes, n = _table(ts)
        _lib.call("sgb_comm_fused_synch_half", self._h, ptrs, sizes, n, int(send), _stream())

    def sparsification(self, t, accumulation, sparsThreshold, topK):
        self.fusedSparsification([t], accumulation, sparsThreshold, topK)

    def fusedSparsification(self, ts, accumulation, sparsThreshold, topK):
        assert ts[0].dtype == torch.float32, "sparsification supports fp32 only"
        ptrs, sizes, n = _table(ts)
        acc = None if accumulation is None else accumulation.data_ptr()
        _lib.call("sgb_comm_sparsification", self._h, ptrs, sizes, n, acc,
                  float(sparsThreshold), int(bool(topK)), _stream())

    def boundedSparsification(self, ts, accumulation, sparsThreshold, capacity):
        """Threshold sparsification with a fixed exchange of `capacity` slots per
        rank and no host wait for the counts (no counterpart in the reference,
        whose fusedSparsification reads them back, communicator.cc:657-669).
        Entries a rank selects beyond `capacity` stay in `accumulation`."""
        assert ts[0].dtype == torch.float32, "sparsification supports fp32 only"
        ptrs, sizes, n = _table(ts)
        acc = None if accumulation is None else accumulation.data_ptr()
        _lib.call("sgb_comm_sparsification_bounded", self._h, ptrs, sizes, n, acc, float(sparsThreshold),
                  int(capacity), _stream())

    def sparseDropped(self):
        """Entries this rank's bounded sparsification calls have held back so far."""
        import ctypes
        out = ctypes.c_ulonglong(0)
        _lib.call("sgb_comm_sparse_dropped", self._h, ctypes.byref(out))
        return int(out.value)

    def wait(self):
        _lib.call("sgb_comm_wait", self._h, _stream())
