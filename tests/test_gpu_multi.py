"""Multi-GPU parity on hardware: needs at least two B200s in one box (skipped otherwise).

Each rank is a child process (one per GPU, NCCL over 127.0.0.1, NVLS off, plain peer loads/stores only); the
checks themselves are in tests/multi_gpu_worker.py.  Failure detection is exercised without faulting a GPU: the
only "failure" is a flag wait that nothing satisfies, which must time out and report."""

from __future__ import annotations

import os
import pathlib
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = pathlib.Path(__file__).resolve().parent / "multi_gpu_worker.py"


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_projection_and_chain_on_two_gpus():
    world = 2
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(WORKER)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=420)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed after 420 s]"
        outputs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out[-4000:]}"
        assert "multi-GPU parity ok" in out
