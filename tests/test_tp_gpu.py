"""Tensor-parallel decode on two GPUs (skipped where fewer are visible): the sharded engines with the
peer-memory all-reduce reproduce the unsharded engine's greedy tokens."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_tp2_matches_single_gpu(cuda):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29731",
           str(ROOT / "tests" / "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "tokens identical" in r.stdout
