"""Peer-memory all-reduce on 2+ GPUs of one node (skipped on a single-GPU box).

The checks themselves live in tests/allreduce_worker.py, launched here as one process per GPU
with torch.distributed.run; NVLS is switched off for NCCL, and the library's own kernel uses
plain peer loads and stores only.
"""
import os
import socket
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_multi_gpu(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "allreduce_worker.py")]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stdout[-4000:]
    for r in range(world):
        assert f"ALLREDUCE_WORKER_OK rank {r}" in res.stdout, res.stdout[-4000:]
