"""Data-parallel training on two GPUs of one node (skipped on a single-GPU box): replicas stay bit-identical, eager and
captured steps both reduce gradients, the loss goes down."""
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_rank_data_parallel_training():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    worker = Path(__file__).resolve().parent / "dp_worker.py"
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", str(port), str(worker)], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "DP_RESULT ok=1" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
