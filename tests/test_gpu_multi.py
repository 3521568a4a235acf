"""Multi-GPU checks (skipped with fewer than two GPUs): peer-memory sharded optimizer."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_adam_over_peer_memory():
    worker = os.path.join(os.path.dirname(__file__), "multi_gpu_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker],
        capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and "MULTI_GPU_OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]
