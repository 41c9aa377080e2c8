"""Communicator parity on real GPUs: world size 1 always, 2 when the box has
two GPUs.  Each run is a fresh set of processes (one per GPU) so that NCCL
state never leaks into the pytest process."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_world(n, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "dist_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    if r.returncode != 0:
        # keep the ranks' own tracebacks, not only the launcher's summary
        lines = [ln for ln in r.stderr.splitlines() if ln.startswith("[rank") or "Error" in ln]
        raise AssertionError("\n".join(lines[-40:]) or r.stderr[-4000:])
    assert r.stdout.count("communicator checks passed") == n, r.stdout[-2000:]


def test_communicator_world_1():
    run_world(1, 29611)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_communicator_world_2():
    run_world(2, 29612)


def test_caller_streams_profiling_and_registration_at_one_rank():
    """The communicator on three caller-owned streams (the reference takes s,
    c1, c2 from the device Context), per-phase timing under the reference's
    operation names, NCCL buffer registration and a CTA cap: one rank, so every
    dense mode must hand back its input (fp16 transport: rounded once)."""
    import ctypes as C

    from singa_b200 import _lib
    from singa_b200.communicator import Communicator, NcclIdHolder
    L = _lib.lib()
    comm = Communicator(torch.cuda.current_device(), 1, NcclIdHolder(), buffSize=1 << 20, max_ctas=8)
    try:
        streams = [torch.cuda.Stream() for _ in range(3)]
        ptrs = [C.c_void_p(s.cuda_stream) for s in streams]
        assert L.sgb_comm_use_streams(comm._h, ptrs[0], ptrs[0], ptrs[2]) == -6        # must be distinct
        assert L.sgb_comm_use_streams(comm._h, *ptrs) == 0
        for w in range(3):
            assert L.sgb_comm_stream(comm._h, w) == streams[w].cuda_stream
        arena = torch.randn(300000, device="cuda")
        comm.register(arena)
        want = arena.clone()
        a, b = arena[:100000], arena[100000:]
        scattered = [torch.randn(5000, device="cuda"), torch.randn(77, device="cuda")]
        want_s = [t.clone() for t in scattered]
        comm.profile_begin()
        comm.fusedSynch([a], send=False)
        comm.fusedSynch([b], send=False)
        comm.fusedSynch([a, b], send=True)                 # contiguous: reduced in place on s
        assert L.sgb_comm_result_stream(comm._h) == streams[2].cuda_stream
        # staged work is pending: the streams cannot be swapped now
        comm.fusedSynch([scattered[0]], send=False)
        assert L.sgb_comm_use_streams(comm._h, *ptrs) == -7                            # SGB_ERR_STATE
        comm.fusedSynch([scattered[1]], send=False)
        comm.fusedSynch(scattered, send=True)              # scattered: packed, unpacked on c1
        assert L.sgb_comm_result_stream(comm._h) == streams[1].cuda_stream
        h = torch.randn(4096, device="cuda")
        want_h = h.half().float()
        comm.synchHalf(h)
        comm.wait()
        rows = comm.profile_end()
        torch.cuda.synchronize()
        assert torch.equal(arena, want)
        assert all(torch.equal(x, y) for x, y in zip(scattered, want_s))
        assert torch.equal(h, want_h)
        names = [r[0] for r in rows]
        assert names.count("Dist_s_fusedSynch_allreduce") == 2
        for expected in ("Dist_c1_fusedSynch_filling", "Dist_c1_fusedSynch_copyBackToTensor",
                         "Dist_c1_synchHalf_float2half", "Dist_s_synchHalf_allreduce", "Dist_c2_synchHalf_half2float"):
            assert expected in names, (expected, names)
        assert all(t1 >= t0 >= 0.0 for _, t0, t1 in rows)
        assert comm.profile_end() == []                    # timing is off again
    finally:
        torch.cuda.synchronize()
        comm.close()
