"""Tensor-parallel decode: one process per GPU (torch.distributed for the rendezvous), each with a Backend
shard (backend.py, tp > 1). This module creates the peer-memory all-reduce state of libie_b200
(csrc/allreduce.cu), exchanges the CUDA-IPC handles, and attaches the state to the shard's engine. From then
on the engine serves the shard's ALLREDUCE stops itself: after every K-split GEMV (attn_output, ffn_down) one
kernel pushes the partial to every rank over NVLink, sums in rank order onto the residual stream and applies
the RMSNorm + Q8 that follows; after the vocabulary-split output head the ranks exchange their local argmax
(value, index) and every rank keeps the best, ties to the smaller index, as one argmax would. A step is the
engine's own CUDA graph, the same on every rank; nothing of it runs in Python.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import check
from .backend import Backend

_vp = C.c_void_p


class TensorParallelBackend:
    def __init__(self, shard: Backend, group):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.b, self.group = torch, dist, shard, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if shard.tp != self.world or shard.rank != self.rank:
            raise ValueError("the shard was built for another rank / degree")
        self.lib = _lib.load()
        self.dev = shard.device
        c = shard.cfg
        h = _vp()
        with torch.cuda.device(self.dev):
            # room for a whole prompt chunk per exchange (T x dim floats), so that a chunk's stop is one launch
            check(self.lib.ie_b200_ar_create(self.rank, self.world, c.dim * max(1, shard.T), C.byref(h)))
            self.ar = h
            blob = (C.c_uint8 * 128)()
            check(self.lib.ie_b200_ar_handles(self.ar, blob))
            mine = torch.tensor(list(bytes(blob)), dtype=torch.uint8, device=self.dev)
            allb = torch.empty(128 * self.world, dtype=torch.uint8, device=self.dev)
            dist.all_gather_into_tensor(allb, mine, group=group)
            raw = (C.c_uint8 * (128 * self.world)).from_buffer_copy(allb.cpu().numpy().tobytes())
            check(self.lib.ie_b200_ar_connect(self.ar, raw))
            check(self.lib.ie_b200_engine_set_collective(shard.h, self.ar, self.rank * shard.vocab_l))
        shard.collective = True
        # capture the step graph (or build the persistent kernel's program) now: the first step should not spend its time on
        # that after the ranks have been aligned (the kernels wait for a peer for 2 s at most)
        _ = shard.launches_per_step

    def _align(self):
        """The kernels' waits for a peer are bounded (2 s): make sure no rank launches long before the others."""
        with self.torch.cuda.device(self.dev):
            self.dist.barrier(group=self.group)

    def step(self, tok: int, pos: int, logits=None) -> int:
        """backend.step for the sharded model: host token in, host token out (identical on every rank). logits: optional
        float32[vocab / world] that receives this rank's slice of the logits."""
        self._align()
        return self.b.step(tok, pos, logits)[0]

    def run(self, toks, pos: int, last_only: bool = True):
        """backend.run for the sharded model: a prompt chunk of up to T tokens at positions pos..; a stop of the chunk is one
        exchange over T x dim floats. Returns the argmax tokens (identical on every rank)."""
        self._align()
        return self.b.run(0, toks, pos, last_only=last_only)

    def decode(self, tok: int, pos: int, K: int, timed: bool = False):
        """K greedy tokens, the argmax fed back on the device. timed: also return the device milliseconds."""
        self._align()
        out, ms = self.b.decode(tok, pos, K)
        return (out, ms) if timed else out

    @property
    def launches_per_step(self) -> int:
        return self.b.launches_per_step

    def describe(self) -> dict:
        n_stops = sum(1 for o in self.b.ops if o.kind == 8)
        return {"kind": "one kernel per stop: push over peer memory (CUDA IPC, 64-bit {epoch, word} stores over NVLink, polled in place), "
                        "sum in rank order + residual + RMSNorm + Q8; bounded waits",
                "calls_per_step": n_stops + 1, "floats_per_call": self.b.cfg.dim, "launches_per_step": self.launches_per_step}

    def close(self):
        self.torch.cuda.synchronize(self.dev)
        if self.ar:
            check(self.lib.ie_b200_engine_set_collective(self.b.h, None, 0))
            self.lib.ie_b200_ar_destroy(self.ar)
            self.ar = None
        self.b.close()
