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
