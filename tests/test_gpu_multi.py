"""Multi-GPU parity (needs >= 2 GPUs, skipped otherwise): expert-parallel MoE and row-sharded dense layers against
the single-GPU result, one NCCL rank per GPU."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expert_parallel_and_row_sharding_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    worker = Path(__file__).resolve().parent / "ep_worker.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29517", str(worker)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
