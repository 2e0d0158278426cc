"""Worker of the tensor-parallel GPU test (launched by torch.distributed.run, one process per GPU): decode the
tiny model sharded over the ranks and compare with the unsharded engine on rank 0's GPU."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from amd_c_b200 import gguf  # noqa: E402
from amd_c_b200.backend import Backend, greedy  # noqa: E402
from amd_c_b200.tp import TensorParallelBackend  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', rank))}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    cfg = gguf.make_model(gguf.config("tiny"), seed=0)
    n_ctx, n_gen, prompt = 96, 24, [1, 2, 3]
    tpb = TensorParallelBackend(Backend(cfg, n_ctx, kv_f32=True, tp=world, rank=rank, device=dev), dist.group.WORLD)
    tok, ids = prompt[0], list(prompt)
    for pos in range(len(prompt) - 1):
        tpb.step(prompt[pos], pos)
    out = tpb.decode(prompt[-1], len(prompt) - 1, n_gen)
    ids += [int(t) for t in out]
    # every rank must hold the same tokens
    t = torch.tensor(ids, dtype=torch.int64, device=dev)
    gathered = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(gathered, t)
    assert all(torch.equal(gathered[0], g) for g in gathered), "ranks disagree on the decoded tokens"
    if rank == 0:
        single = Backend(cfg, n_ctx, kv_f32=True, device=dev)
        want = greedy(single, prompt, n_gen)
        single.close()
        # the cross-rank sum changes the float order of two sums per layer, so a near-tie may flip: require a
        # long common prefix and report it
        common = next((i for i, (a, b) in enumerate(zip(ids, want)) if a != b), len(want))
        print(f"TP{world}: {common} of {len(want)} tokens identical to the unsharded engine", flush=True)
        assert common >= len(prompt) + 8, (ids, want)
    tpb.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
