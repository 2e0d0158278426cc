"""Host side of the decode path above the C ABI: the Python mirror of the
reference's backend interface (src/backend.h:7-49 of amd-infer) and of the
part of its graph builder that llama / qwen2 models use
(src/model.c:1321-1381, :1518-1575).

`Backend` owns one ie_b200_engine (one GPU). `step`, `run`, `accept`,
`read_rows`, `copy_rows`, `close` have the reference's meaning; errors raise
IeB200Error where the reference exits with a message. With `tp > 1` the
matrices are sharded Megatron-style (q/k/v/gate/up by rows, o/down by
columns, the output head by vocabulary rows) and the op list gains ALLREDUCE
stops that `TensorParallelBackend` (tp.py) serves with collectives.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import GGML_TO_MAT, MAT_F32, check
from .gguf import ModelConfig
from .synth import GGML_F32, GGML_Q4_0, GGML_Q4_K, GGML_Q6_K, GGML_Q8_0

NONE = 0xFFFFFFFFFFFFFFFF
OP_EMBED, OP_RMSNORM, OP_QUANT, OP_GEMV, OP_ROPE_KV, OP_ATTN, OP_SWIGLU, OP_ARGMAX, OP_ALLREDUCE, OP_ADD = range(10)


Op, EngineDesc = _lib.Op, _lib.EngineDesc
_vp, _u32, _u64, _int = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def q8_bytes(nb: int) -> int:
    return 40 * nb


@dataclass
class Buf:
    """An arena buffer: byte offset of token 0 and the stride between token rows (the reference's `buf`, src/model.h:289-294)."""
    name: str
    off: int
    stride: int


def rope_tables(n_ctx: int, n_rot: int, base: float):
    """theta = p * base^(-2 i / n_rot) in double; cos and sin cast to float (src/model.c:1655-1664)."""
    i = np.arange(n_rot // 2, dtype=np.float64)
    inv = np.power(np.float64(np.float32(base)), -2.0 * i / float(n_rot))
    th = np.arange(n_ctx, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(th).astype(np.float32), np.sin(th).astype(np.float32)


def shard_rows(raw: np.ndarray, typ: int, rows: int, cols: int, r0: int, r1: int) -> np.ndarray:
    """Rows [r0, r1) of a GGUF tensor (its rows are contiguous)."""
    per = raw.reshape(-1).size // rows
    return raw.reshape(-1)[r0 * per: r1 * per]


def shard_cols(raw, typ: int, rows: int, cols: int, c0: int, c1: int):
    """Columns [c0, c1) of a GGUF tensor: whole 32-blocks (Q4_0) or 256 super-blocks (K kinds). Works on numpy or torch uint8."""
    gran, bb = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210), GGML_F32: (1, 4)}[typ]
    if c0 % gran or c1 % gran:
        raise ValueError(f"column split [{c0}, {c1}) is not a multiple of the {gran}-weight block of GGML type {typ}")
    v = raw.reshape(rows, cols // gran, bb)
    return v[:, c0 // gran: c1 // gran, :]


class Backend:
    """One GPU's decode backend for a llama / qwen2 ModelConfig.

    device_tensors: optional name -> (ggml_type, rows, cols, torch uint8 CUDA tensor of GGUF bytes) for matrices
    generated on the device; all other tensors come from cfg.tensors (numpy). kv_f32: float KV cache (the reference CPU backend's precision).
    tp / rank: tensor-parallel degree and this engine's slice.
    step_mode: "graph" (a CUDA graph of one kernel per op: the library's default), "kernel" (the persistent step kernel, an error
    where it cannot run), "auto" (the kernel where it can run, else the graph); None leaves the library's default (graph, or what
    IE_B200_STEP says).
    """

    STEP_MODES = {"auto": 0, "graph": 1, "kernel": 2}

    def __init__(self, cfg: ModelConfig, n_ctx: int, T: int = 1, kv_f32: bool = False, device_tensors: dict | None = None, tp: int = 1,
                 rank: int = 0, device=None, step_mode: str | None = None):
        import torch

        _lib.require_gpu()
        self.lib = _lib.load()
        self.torch = torch
        self.cfg, self.n_ctx, self.T, self.tp, self.rank = cfg, n_ctx, max(1, T), tp, rank
        self.collective = False  # set once an all-reduce state is attached to the engine (tp.py)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if cfg.n_head % tp or cfg.n_kv % tp or cfg.ffn % (32 * tp) or cfg.vocab % tp:
            raise ValueError(f"tp={tp} does not divide heads {cfg.n_head}/{cfg.n_kv}, ffn {cfg.ffn} or vocab {cfg.vocab}")
        self.nh, self.nkv, self.hd = cfg.n_head // tp, cfg.n_kv // tp, cfg.hd
        self.ffn_l, self.vocab_l = cfg.ffn // tp, cfg.vocab // tp
        self._keep = []  # device tensors the engine points into
        self._dev = device_tensors or {}
        self._plan_buffers()
        d = EngineDesc(self.nh, self.nkv, self.hd, n_ctx, cfg.n_layer, self.T, self.vocab_l, cfg.eps, int(cfg.neox), int(kv_f32),
                       self.arena_bytes, self.bufs["logits"].off, self.bufs["argmax"].off, self.bufs["logits"].stride,
                       self.bufs["argmax"].stride)
        h = _vp()
        d.vocab = cfg.vocab  # token ids are checked against the full vocabulary even when the head is sharded
        with torch.cuda.device(self.device):
            check(self.lib.ie_b200_engine_create(C.byref(d), C.byref(h)))
            self.h = h
            cs, sn = rope_tables(n_ctx, self.hd, cfg.rope_base)
            check(self.lib.ie_b200_engine_set_rope(self.h, cs.ctypes.data_as(_vp), sn.ctypes.data_as(_vp)))
            self._build_ops()
            if step_mode is not None:
                check(self.lib.ie_b200_engine_set_step_mode(self.h, self.STEP_MODES[step_mode]))
        self.weight_bytes_per_token = int(self.lib.ie_b200_engine_weight_bytes_per_token(self.h))
        self.all_logits = 0
        self.verify_max = 0

    # ---- arena -------------------------------------------------------------
    def _plan_buffers(self):
        c = self.cfg
        qd, kvd = self.nh * self.hd, self.nkv * self.hd
        sizes = [("x", c.dim * 4), ("xn", c.dim * 4), ("xq", q8_bytes(c.dim // 32)), ("qkv", (qd + 2 * kvd) * 4), ("att", qd * 4),
                 ("attq", q8_bytes(qd // 32)), ("gu", 2 * self.ffn_l * 4), ("h", self.ffn_l * 4), ("guq", q8_bytes(self.ffn_l // 32)), ("part", c.dim * 4),
                 ("logits", self.vocab_l * 4), ("argmax", 8)]
        self.bufs, off = {}, 0
        for name, n in sizes:
            stride = _align(n)
            self.bufs[name] = Buf(name, off, stride)
            off += stride * self.T
        self.arena_bytes = off

    # ---- weights -----------------------------------------------------------
    def _to_device(self, raw):
        torch = self.torch
        if isinstance(raw, np.ndarray):
            return torch.from_numpy(np.ascontiguousarray(raw).reshape(-1)).to(self.device)
        return raw.contiguous().reshape(-1)

    def _add_mat(self, parts, interleave: bool = False) -> int:
        """parts: list of (ggml_type, rows, cols, raw bytes) with one type and column count: stacked by rows into one matrix.
        interleave (two parts of equal row count): rows alternate part 0, part 1 (gate_i, up_i), so that the warp that owns a
        row pair of the GEMV owns one SwiGLU output."""
        torch = self.torch
        typ, cols = parts[0][0], parts[0][2]
        kind = GGML_TO_MAT[typ]
        rows = sum(p[1] for p in parts)
        rowb = self.lib.ie_b200_row_bytes(kind, cols)
        buf = torch.empty(max(16, rows * rowb), dtype=torch.uint8, device=self.device)
        r = 0
        st = torch.cuda.current_stream(self.device).cuda_stream
        for _, pr, _, raw in parts:
            src = self._to_device(raw)
            check(self.lib.ie_b200_repack_gguf(typ, src.data_ptr(), pr, cols, buf.data_ptr() + r * rowb, st))
            r += pr
        torch.cuda.current_stream(self.device).synchronize()
        if interleave:
            half = rows // 2
            two = buf[: rows * rowb].view(2, half, rowb)
            buf = torch.stack((two[0], two[1]), dim=1).reshape(-1).contiguous()
        self._keep.append(buf)
        h = self.lib.ie_b200_engine_add_mat_device(self.h, kind, rows, cols, buf.data_ptr())
        if h < 0:
            check(h)
        return h

    def _add_vec(self, v: np.ndarray) -> int:
        v = np.ascontiguousarray(v, dtype=np.float32)
        h = self.lib.ie_b200_engine_add_vec(self.h, v.ctypes.data_as(_vp), v.size)
        if h < 0:
            check(h)
        return h

    def _vec(self, name: str) -> np.ndarray:
        return self.cfg.tensors[name].f32()

    def _tensor(self, name: str):
        """(ggml_type, rows, cols, bytes): bytes are a torch CUDA tensor (device_tensors) or a numpy array (cfg.tensors)."""
        if name in self._dev:
            return self._dev[name]
        t = self.cfg.tensors[name]
        return t.ggml_type, t.rows, t.cols, t.raw()

    def _rows(self, name: str, r0: int, r1: int):
        typ, rows, cols, raw = self._tensor(name)
        per = raw.reshape(-1).shape[0] // rows
        return typ, r1 - r0, cols, raw.reshape(-1)[r0 * per: r1 * per]

    def _cols(self, name: str, c0: int, c1: int):
        typ, rows, cols, raw = self._tensor(name)
        sub = shard_cols(raw, typ, rows, cols, c0, c1)
        sub = np.ascontiguousarray(sub) if isinstance(sub, np.ndarray) else sub.contiguous()
        return typ, rows, c1 - c0, sub

    # ---- the op list ---------------------------------------------------------
    def _op(self, kind, a=None, b=None, c=None, qo=None, res=None, mat=-1, vec=-1, layer=-1, n=0, nh=0, aoff=0, boff=0, coff=0):
        def o(buf, extra=0):
            return (NONE, 0) if buf is None else (self.bufs[buf].off + extra, self.bufs[buf].stride)

        (ao, as_), (bo, bs), (co, cs), (qoo, qs), (ro, rs) = o(a, aoff), o(b, boff), o(c, coff), o(qo), o(res)
        self.ops.append(Op(kind, mat, vec, layer, n, nh, ao, bo, co, qoo, ro, as_, bs, cs, qs, rs))

    def _gemv_group(self, names_rows, x_q8: str, x_f32: str, out: str, bias_names=None, interleave: bool = False) -> bool:
        """GEMVs of several row slices into one output buffer: merged into one matrix when the kinds agree
        (as the reference merges q/k/v and gate/up, src/model.c:882-887), else one GEMV per part at its offset."""
        parts = [self._rows(n, r0, r1) for n, r0, r1 in names_rows]
        bias = None
        if bias_names:
            bias = np.concatenate([self._vec(n)[r0:r1] for (n, r0, r1) in bias_names])
        if len({p[0] for p in parts}) == 1:
            f32 = parts[0][0] == GGML_F32
            il = interleave and not f32 and len(parts) == 2 and parts[0][1] == parts[1][1] and bias is None
            m = self._add_mat(parts, interleave=il)
            self._op(OP_GEMV, a=x_f32 if f32 else x_q8, b=out, mat=m, vec=self._add_vec(bias) if bias is not None else -1, n=parts[0][2])
            return il
        off = 0
        for p in parts:
            m = self._add_mat([p])
            f32 = p[0] == GGML_F32
            v = self._add_vec(bias[off: off + p[1]]) if bias is not None else -1
            self._op(OP_GEMV, a=x_f32 if f32 else x_q8, b=out, boff=off * 4, mat=m, vec=v, n=p[2])
            off += p[1]
        return False

    def _build_ops(self):
        c, tp, r = self.cfg, self.tp, self.rank
        self.ops = []
        qd, kvd = self.nh * self.hd, self.nkv * self.hd
        q0, k0 = r * qd, r * kvd  # this rank's first q / kv row
        f0 = r * self.ffn_l
        emb = self._add_mat([self._tensor("token_embd.weight")])
        self._op(OP_EMBED, a="x", mat=emb, n=c.dim)
        self._op(OP_RMSNORM, a="x", b="xn", qo="xq", vec=self._add_vec(self._vec("blk.0.attn_norm.weight")), n=c.dim)
        for l in range(c.n_layer):
            p = f"blk.{l}."
            bias = [(p + "attn_q.bias", q0, q0 + qd), (p + "attn_k.bias", k0, k0 + kvd), (p + "attn_v.bias", k0, k0 + kvd)] if c.qkv_bias else None
            self._gemv_group([(p + "attn_q.weight", q0, q0 + qd), (p + "attn_k.weight", k0, k0 + kvd), (p + "attn_v.weight", k0, k0 + kvd)],
                             "xq", "xn", "qkv", bias)
            self._op(OP_ROPE_KV, a="qkv", b="qkv", c="qkv", boff=qd * 4, coff=(qd + kvd) * 4, layer=l, n=qd, nh=self.nh)
            self._op(OP_ATTN, a="qkv", b="att", qo="attq", layer=l, n=qd)
            wo = self._add_mat([self._cols(p + "attn_output.weight", q0, q0 + qd)])
            nxt_norm = self._add_vec(self._vec(p + "ffn_norm.weight"))
            if tp == 1:
                self._op(OP_GEMV, a="attq", b="x", res="x", mat=wo, n=qd)
                self._op(OP_RMSNORM, a="x", b="xn", qo="xq", vec=nxt_norm, n=c.dim)
            else:
                self._op(OP_GEMV, a="attq", b="part", mat=wo, n=qd)
                self._op(OP_ALLREDUCE, a="part", c="x", n=c.dim)  # x = x + sum over ranks of part
                self._op(OP_RMSNORM, a="x", b="xn", qo="xq", vec=nxt_norm, n=c.dim)
            il = self._gemv_group([(p + "ffn_gate.weight", f0, f0 + self.ffn_l), (p + "ffn_up.weight", f0, f0 + self.ffn_l)], "xq", "xn", "gu",
                                  interleave=self.ffn_l % 32 == 0)
            if il:  # gate_i / up_i in alternating rows: gu holds the pairs, h = silu(gate) * up; one token folds it into the GEMV
                self._op(OP_SWIGLU, a="gu", b="h", qo="guq", n=self.ffn_l, nh=1)
            else:
                self._op(OP_SWIGLU, a="gu", b="gu", boff=self.ffn_l * 4, qo="guq", n=self.ffn_l)
            wd = self._add_mat([self._cols(p + "ffn_down.weight", f0, f0 + self.ffn_l)])
            nname = f"blk.{l + 1}.attn_norm.weight" if l + 1 < c.n_layer else "output_norm.weight"
            nxt_norm = self._add_vec(self._vec(nname))
            if tp == 1:
                self._op(OP_GEMV, a="guq", b="x", res="x", mat=wd, n=self.ffn_l)
                self._op(OP_RMSNORM, a="x", b="xn", qo="xq", vec=nxt_norm, n=c.dim)
            else:
                self._op(OP_GEMV, a="guq", b="part", mat=wd, n=self.ffn_l)
                self._op(OP_ALLREDUCE, a="part", c="x", n=c.dim)
                self._op(OP_RMSNORM, a="x", b="xn", qo="xq", vec=nxt_norm, n=c.dim)
        self.i_head = len(self.ops)
        v0 = r * self.vocab_l
        head = self._rows("output.weight" if ("output.weight" in c.tensors or "output.weight" in self._dev) else "token_embd.weight", v0,
                          v0 + self.vocab_l)
        m = self._add_mat([head])
        self._op(OP_GEMV, a="xn" if head[0] == GGML_F32 else "xq", b="logits", mat=m, n=c.dim)
        self._op(OP_ARGMAX, a="logits", b="argmax", n=self.vocab_l)
        arr = (Op * len(self.ops))(*self.ops)
        check(self.lib.ie_b200_engine_set_ops(self.h, arr, len(self.ops), self.i_head))

    # ---- the backend interface (src/backend.h:7-49) ----------------------------
    def step(self, tok: int, pos: int, logits: np.ndarray | None = None):
        """One decode step; returns (argmax token, device milliseconds). logits: optional float32[vocab] to fill."""
        if self.tp != 1 and not self.collective:
            raise _lib.IeB200Error("a tensor-parallel shard needs its collective first (TensorParallelBackend attaches it)")
        nxt, ms = _u32(0), C.c_double(0)
        lp = logits.ctypes.data_as(_vp) if logits is not None else None
        with self.torch.cuda.device(self.device):
            check(self.lib.ie_b200_engine_step(self.h, tok, pos, lp, C.byref(nxt), C.byref(ms)))
        return int(nxt.value), ms.value

    def run(self, sec: int, toks, pos: int, last_only: bool = True, want_prob: bool = False):
        """T tokens at positions pos..pos+T-1 (a prompt chunk); returns the T argmax tokens (and probabilities)."""
        if sec != 0:
            raise _lib.IeB200Error(f"run: section {sec} is not built (only the model, section 0)")
        if self.tp != 1 and not self.collective:
            raise _lib.IeB200Error("a tensor-parallel shard needs its collective first (TensorParallelBackend attaches it)")
        toks = np.ascontiguousarray(toks, dtype=np.uint32)
        out = np.zeros(toks.size, np.uint32)
        prob = np.zeros(toks.size, np.float32) if want_prob else None
        with self.torch.cuda.device(self.device):
            check(self.lib.ie_b200_engine_run(self.h, toks.ctypes.data_as(_vp), toks.size, pos, int(last_only), out.ctypes.data_as(_vp),
                                              prob.ctypes.data_as(_vp) if want_prob else None))
        return (out, prob) if want_prob else out

    def decode(self, tok: int, pos: int, K: int):
        """K greedy tokens with the argmax fed back on the device (no host round trip per token).
        Returns (tokens uint32[K], device milliseconds)."""
        if self.tp != 1 and not self.collective:
            raise _lib.IeB200Error("a tensor-parallel shard needs its collective first (TensorParallelBackend attaches it)")
        out, ms = np.zeros(K, np.uint32), C.c_double(0)
        with self.torch.cuda.device(self.device):
            check(self.lib.ie_b200_engine_decode(self.h, tok, pos, K, out.ctypes.data_as(_vp), C.byref(ms)))
        return out, ms.value

    def accept(self, k: int) -> None:
        """No recurrent state in llama / qwen2: nothing to roll back (src/backend.h:24)."""

    def read_rows(self, name: str, r0: int, n: int) -> np.ndarray:
        """n token rows of buffer `name` from row r0, as raw bytes [n, stride]."""
        b = self.bufs[name]
        dst = np.zeros((n, b.stride), np.uint8)
        check(self.lib.ie_b200_engine_read_rows(self.h, b.off, b.stride, r0, n, dst.ctypes.data_as(_vp)))
        return dst

    def copy_rows(self, dst: str, d0: int, src: str | None, r0: int, n: int) -> None:
        d = self.bufs[dst]
        s = self.bufs[src] if src is not None else d
        check(self.lib.ie_b200_engine_copy_rows(self.h, d.off, d.stride, d0, s.off, s.stride, r0, n, min(d.stride, s.stride), int(src is None)))

    @property
    def step_is_kernel(self) -> bool:
        """Whether one-token steps run as the persistent step kernel (one launch per step or per decode call)."""
        with self.torch.cuda.device(self.device):
            return bool(self.lib.ie_b200_engine_step_is_kernel(self.h))

    PHASE_KINDS = ("embed", "gemv", "attention", "merge", "argmax", "finish", "reduce", "argmax_exchange", "gemv_from_q8", "gemv_with_norm",
                   "gemv_with_swiglu", "gemv_same_activations")

    def phase_times(self, enable: bool = True) -> dict:
        """Per phase kind of the persistent step kernel: {kind: (work ms, barrier ms, barriers)} summed by CTA 0 since the last call."""
        buf = (C.c_double * 36)()
        check(self.lib.ie_b200_engine_phase_times(self.h, int(enable), buf))
        return {k: (buf[3 * i], buf[3 * i + 1], int(buf[3 * i + 2])) for i, k in enumerate(self.PHASE_KINDS) if buf[3 * i + 2]}

    def clear_error(self) -> None:
        check(self.lib.ie_b200_engine_clear_error(self.h))

    @property
    def launches_per_step(self) -> int:
        return int(self.lib.ie_b200_engine_launches_per_step(self.h))

    def enqueue_kinds(self, first: int, last: int, kind_mask: int, stream: int, T: int = 1) -> None:
        """Enqueue the ops [first, last) whose kind bit is in kind_mask on a CUDA stream (no input upload, no sync)."""
        check(self.lib.ie_b200_engine_enqueue_kinds(self.h, first, last, kind_mask, T, stream))

    def set_input(self, toks, pos: int, stream: int) -> None:
        t = np.ascontiguousarray(toks, dtype=np.uint32)
        check(self.lib.ie_b200_engine_set_input(self.h, t.ctypes.data_as(_vp), t.size, pos, stream))

    def run_ops(self, tok: int, pos: int, last_op: int) -> None:
        """Debug aid for parity tests: ops [0, last_op) of one token, synchronously (no graph)."""
        t = np.array([tok], np.uint32)
        st = self.torch.cuda.current_stream(self.device)
        with self.torch.cuda.device(self.device):
            check(self.lib.ie_b200_engine_set_input(self.h, t.ctypes.data_as(_vp), 1, pos, st.cuda_stream))
            check(self.lib.ie_b200_engine_enqueue(self.h, 0, last_op, 1, st.cuda_stream))
        st.synchronize()

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.ie_b200_engine_destroy(self.h)
            self.h = None
            self._keep.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def prefill(b: Backend, prompt, chunk: int = 256) -> int:
    """The prompt in chunks of up to `chunk` tokens; returns the first generated token
    (the role of prefill() in the reference's src/gen.c:139)."""
    prompt = np.asarray(prompt, dtype=np.uint32)
    first = 0
    for p0 in range(0, prompt.size, chunk):
        part = prompt[p0: p0 + chunk]
        out = b.run(0, part, p0, last_only=True)
        first = int(out[-1])
    return first


def greedy(b: Backend, prompt, n_gen: int, use_prefill: bool = False, chunk: int = 256):
    """Greedy decode as ie-run does (src/main.c:192-225): returns prompt + generated ids."""
    prompt = [int(t) for t in prompt]
    ids = list(prompt)
    if use_prefill:
        tok = prefill(b, prompt, chunk)
        pos = len(prompt)
        ids.append(tok)
        n_left = n_gen - 1
    else:
        tok, pos, n_left = prompt[0], 0, n_gen
    total = len(prompt) + n_gen
    while len(ids) < total:
        nxt, _ = b.step(tok, pos)
        pos += 1
        if pos < len(prompt):
            tok = prompt[pos]
        else:
            tok = nxt
            ids.append(nxt)
    return ids
