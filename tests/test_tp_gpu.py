"""Tensor-parallel decode on 2, 4 and 8 GPUs (skipped where fewer are visible): the sharded engines, in both step modes
(CUDA graph of one kernel per op with the one-kernel all-reduce + norm stop; persistent step kernel with the exchange
inside it), against the unsharded engine: logits of the first steps, identical tokens on every rank."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["graph", "kernel"])
def test_tp_matches_single_gpu(cuda, world, mode):
    import torch

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port",
           str(29731 + world), str(ROOT / "tests" / "tp_worker.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "chained tokens identical" in r.stdout
    print(r.stdout[-300:])
