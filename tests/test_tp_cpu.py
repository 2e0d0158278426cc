"""The host logic of the tensor-parallel path on CPU: two gloo ranks shard a Q4_0 matrix the way backend.py
does (rows for q/k/v/gate/up/head, whole 32-column blocks for o/down), run the oracle GEMV on their shards and
exchange the partial sums; the result must equal the unsharded GEMV (rows: bit for bit; columns: to rounding,
because the cross-rank sum changes the float order)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from amd_c_b200 import synth  # noqa: E402
from amd_c_b200.backend import shard_cols, shard_rows  # noqa: E402


def _worker(rank: int, world: int, port: int, q):
    import torch

    from oracle.oracle import Oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ora = Oracle()
    rng = np.random.default_rng(5)  # the same seed on every rank: the same full matrix
    rows, cols = 96, 1024
    raw = synth.q4_0_normal(rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    kind, qw, qs = ora.repack(synth.GGML_Q4_0, raw, rows, cols)
    full = ora.gemv(kind, qw, qs, rows, cols, ora.quant_q8(x))
    # row split: this rank's rows, all-gathered
    r0, r1 = rank * rows // world, (rank + 1) * rows // world
    sub = shard_rows(raw, synth.GGML_Q4_0, rows, cols, r0, r1)
    k2, w2, s2 = ora.repack(synth.GGML_Q4_0, sub, r1 - r0, cols)
    mine = torch.from_numpy(ora.gemv(k2, w2, s2, r1 - r0, cols, ora.quant_q8(x)))
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    row_ok = bool((torch.cat(parts).numpy().view(np.uint32) == full.view(np.uint32)).all())
    # column split: this rank's 32-blocks and the matching slice of the Q8 activations (per-32 blocks are shard-local)
    c0, c1 = rank * cols // world, (rank + 1) * cols // world
    subc = np.ascontiguousarray(shard_cols(raw, synth.GGML_Q4_0, rows, cols, c0, c1))
    k3, w3, s3 = ora.repack(synth.GGML_Q4_0, subc, rows, c1 - c0)
    part = torch.from_numpy(ora.gemv(k3, w3, s3, rows, c1 - c0, ora.quant_q8(x[c0:c1])))
    dist.all_reduce(part)
    col_err = float(np.abs(part.numpy() - full).max() / np.abs(full).max())
    if rank == 0:
        q.put((row_ok, col_err))
    dist.destroy_process_group()


def test_sharded_gemv_equals_full_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29641, q)) for r in range(2)]
    for p in procs:
        p.start()
    row_ok, col_err = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert row_ok
    assert col_err <= 1e-5


def test_column_split_granularity():
    raw = np.zeros((4, 2, 144), np.uint8)  # Q4_K: two super-blocks of 256 columns per row
    assert shard_cols(raw, synth.GGML_Q4_K, 4, 512, 0, 256).shape == (4, 1, 144)
    with pytest.raises(ValueError, match="256"):
        shard_cols(raw, synth.GGML_Q4_K, 4, 512, 0, 128)
    q4 = np.zeros((4, 16, 18), np.uint8)
    assert shard_cols(q4, synth.GGML_Q4_0, 4, 512, 128, 384).shape == (4, 8, 18)
