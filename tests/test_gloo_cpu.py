"""Multi-rank behaviour on CPU (Gloo): failures injected on the host reach every rank, the
context-parallel batch transport, and context-parallel training against one group."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _run(case, ranks, port):
    env = dict(os.environ, PYTHONPATH=str(ROOT), AGB200_DISABLE_NATIVE="1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           str(ROOT / "tests" / "gloo_worker.py"), case]
    done = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and f"CASE_OK {case}" in done.stdout, done.stdout[-2000:] + done.stderr[-4000:]


@pytest.mark.parametrize("case,ranks,port", [
    ("fetch_error_reaches_every_rank", 3, 29641),
    ("uneven_end_stops_everyone", 2, 29642),
    ("cp_transport_shares_batch_and_rng", 4, 29643),
    ("cp_prepare_error_reaches_the_group", 2, 29644),
    ("context_parallel_matches_single_group", 2, 29645),
    ("node_groups_for_hybrid_sharding", 4, 29646),
    ("kernel_status_of_one_rank_stops_every_rank", 2, 29647),
    ("a_rank_that_leaves_ends_the_next_collective_of_the_others", 3, 29648),
])
def test_gloo_case(case, ranks, port):
    _run(case, ranks, port)
