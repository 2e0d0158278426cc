"""Tensor-parallel decode: one process per GPU (torch.distributed for the rendezvous), each with a Backend
shard (backend.py, tp > 1). The op list of a shard stops at ALLREDUCE ops; this module runs the segments in
between and serves each stop with the peer-memory all-reduce kernel of libie_b200 (csrc/allreduce.cu): the
partial of the K-split GEMV is pushed to every rank over NVLink and summed in rank order onto the residual stream. The output head is split by vocabulary rows: every rank takes its
local argmax and the (value, index) pairs are all-gathered; ties go to the smaller index, as one argmax would.

A step is captured once into a CUDA graph per rank (segments, all-reduce kernels, the small selection ops) and
replayed; token and position travel through the engine's device scalars.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check
from .backend import OP_ALLREDUCE, Backend

_vp = C.c_void_p


class _DevView:
    """A device address range as a __cuda_array_interface__ object, so torch can wrap engine memory."""

    def __init__(self, ptr: int, n: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3}


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
        # ---- the all-reduce state: create, exchange IPC handles, connect
        h = _vp()
        with torch.cuda.device(self.dev):
            check(self.lib.ie_b200_ar_create(self.rank, self.world, c.dim, C.byref(h)))
            self.ar = h
            blob = (C.c_uint8 * 128)()
            check(self.lib.ie_b200_ar_handles(self.ar, blob))
            mine = torch.tensor(list(bytes(blob)), dtype=torch.uint8, device=self.dev)
            allb = torch.empty(128 * self.world, dtype=torch.uint8, device=self.dev)
            dist.all_gather_into_tensor(allb, mine, group=group)
            raw = (C.c_uint8 * (128 * self.world)).from_buffer_copy(allb.cpu().numpy().tobytes())
            check(self.lib.ie_b200_ar_connect(self.ar, raw))
        # ---- torch views of engine memory
        arena = self.lib.ie_b200_engine_arena(shard.h)
        self.arena_ptr = arena
        Tm = shard.T
        self.scalars = torch.as_tensor(_DevView(self.lib.ie_b200_engine_input_scalars(shard.h), 2 * Tm + 1, "<i4"), device=self.dev)
        lb, ab = shard.bufs["logits"], shard.bufs["argmax"]
        self.logits = torch.as_tensor(_DevView(arena + lb.off, shard.vocab_l, "<f4"), device=self.dev)
        self.argmax = torch.as_tensor(_DevView(arena + ab.off, 2, "<i4"), device=self.dev)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.dev)
        # ---- segments between the ALLREDUCE stops
        self.stops = [i for i, o in enumerate(shard.ops) if o.kind == OP_ALLREDUCE]
        self.hist = torch.zeros(4096, dtype=torch.int64, device=self.dev)
        self.count = torch.zeros(1, dtype=torch.int64, device=self.dev)
        self.pair_v = torch.empty(self.world, dtype=torch.float32, device=self.dev)
        self.pair_i = torch.empty(self.world, dtype=torch.int64, device=self.dev)
        self.stream = torch.cuda.Stream(device=self.dev)
        self.graph = None
        self.launches_per_step = 0

    # ---- one step's work on the current stream (capturable)
    def _enqueue_step(self):
        torch, dist, b = self.torch, self.dist, self.b
        st = torch.cuda.current_stream(self.dev).cuda_stream
        first = 0
        for s in self.stops + [len(b.ops)]:
            check(self.lib.ie_b200_engine_enqueue(b.h, first, s, 1, st))
            if s < len(b.ops):
                o = b.ops[s]
                part, x = self.arena_ptr + o.a, self.arena_ptr + o.c  # x = x + sum over ranks of part
                check(self.lib.ie_b200_ar_allreduce_add(self.ar, part, x, x, o.n, self.err.data_ptr(), st))
            first = s + 1
        # the global argmax: (value, global index) of every rank, ties to the smaller index
        idx = self.argmax[0:1].to(torch.int64)
        val = self.logits.index_select(0, idx)
        dist.all_gather_into_tensor(self.pair_v, val, group=self.group)
        dist.all_gather_into_tensor(self.pair_i, idx + self.rank * b.vocab_l, group=self.group)
        best = torch.where(self.pair_v == self.pair_v.max(), self.pair_i, torch.full_like(self.pair_i, 1 << 40)).min().reshape(1)
        # feed it back: next token, positions + 1, history
        self.hist.index_copy_(0, self.count % 4096, best)
        self.count += 1
        self.scalars[0:1] = best.to(torch.int32)
        self.scalars[b.T:] += 1

    def _ensure_graph(self, tok: int, pos: int):
        if self.graph is not None:
            return
        torch = self.torch
        with torch.cuda.device(self.dev), torch.cuda.stream(self.stream):
            self._set_input(tok, pos)  # the warm pass is the real first step: what it writes (KV row) is what the replay rewrites
            before = self.lib.ie_b200_launch_count()
            self._enqueue_step()  # uncaptured: communicator set-up and other lazy initialisations happen outside the capture
            self.launches_per_step = int(self.lib.ie_b200_launch_count() - before)
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                self._enqueue_step()
            self.graph = g

    def _set_input(self, tok: int, pos: int):
        t = np.array([tok], np.uint32)
        check(self.lib.ie_b200_engine_set_input(self.b.h, t.ctypes.data_as(_vp), 1, pos, self.stream.cuda_stream))
        self.count.zero_()

    def _check_err(self):
        e = int(self.err.item())
        if e:
            raise _lib.IeB200Error(f"a kernel gave up a bounded wait (device error word {e}): a rank is missing or stalled")

    def step(self, tok: int, pos: int) -> int:
        """backend.step for the sharded model: host token in, host token out (identical on every rank)."""
        return int(self.decode(tok, pos, 1)[0])

    def decode(self, tok: int, pos: int, K: int, timed: bool = False):
        """K greedy tokens, the argmax fed back on the device. timed: also return the device milliseconds."""
        torch = self.torch
        if K > 4096:
            raise ValueError("at most 4096 steps per call")
        self._ensure_graph(tok, pos)
        with torch.cuda.device(self.dev), torch.cuda.stream(self.stream):
            self._set_input(tok, pos)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(K):
                self.graph.replay()
            e1.record(self.stream)
            self.stream.synchronize()
            out = self.hist[:K].cpu().numpy().astype(np.uint32)
        self._check_err()
        return (out, e0.elapsed_time(e1)) if timed else out

    def describe(self) -> dict:
        return {"kind": "one-shot push over peer memory (CUDA IPC, plain stores over NVLink), summed in rank order, bounded waits",
                "calls_per_step": len(self.stops), "floats_per_call": self.b.cfg.dim, "launches_per_step": self.launches_per_step}

    def close(self):
        self.graph = None
        self.torch.cuda.synchronize(self.dev)
        if self.ar:
            self.lib.ie_b200_ar_destroy(self.ar)
            self.ar = None
        self.b.close()
