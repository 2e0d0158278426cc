"""Thin torch-tensor wrappers over the kernel-level C ABI.

torch is used for device memory and streams only; every computation is a
call into libie_b200.so on the current torch CUDA stream.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import GGML_TO_MAT, MAT_F32, MAT_Q4, MAT_Q4K, MAT_Q6K, MAT_Q8, check


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def q8_bytes(nb: int) -> int:
    """Bytes of a Q8 activation buffer of nb blocks (int8 x 32 | f32 d | u32 asum)."""
    return 40 * nb


class Mat:
    """A weight matrix in the streaming layout on the device."""

    def __init__(self, kind: int, rows: int, cols: int, data: torch.Tensor):
        self.kind, self.rows, self.cols, self.data = kind, rows, cols, data

    @property
    def nb(self) -> int:
        return self.cols // 32

    @property
    def algorithmic_bytes(self) -> int:
        """Bytes one GEMV must read: 18 B per Q4_0 / Q4_K block, 34 B per Q8_0 block, 26.25 B per
        Q6_K block, 4 B per f32 weight."""
        if self.kind == MAT_F32:
            return self.rows * self.cols * 4
        per = {MAT_Q4: 18.0, MAT_Q8: 34.0, MAT_Q4K: 18.0, MAT_Q6K: 26.25}[self.kind]
        return int(self.rows * self.nb * per)

    @staticmethod
    def from_gguf(ggml_type: int, raw: torch.Tensor, rows: int, cols: int) -> "Mat":
        """raw: uint8 CUDA tensor of the GGUF tensor bytes."""
        lib = _lib.load()
        kind = GGML_TO_MAT[ggml_type]
        nbytes = lib.ie_b200_mat_bytes(kind, rows, cols)
        dst = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=raw.device)
        check(lib.ie_b200_repack_gguf(ggml_type, raw.data_ptr(), rows, cols, dst.data_ptr(), _stream()))
        return Mat(kind, rows, cols, dst)

    @staticmethod
    def from_ref(kind: int, qw: torch.Tensor, qs: torch.Tensor | None, rows: int, cols: int) -> "Mat":
        """qw / qs: the reference loader's repacked arrays (or the f32 weights in qw), on the device."""
        lib = _lib.load()
        nbytes = lib.ie_b200_mat_bytes(kind, rows, cols)
        dst = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=qw.device)
        check(lib.ie_b200_repack_ref(kind, qw.data_ptr(), _p(qs), rows, cols, dst.data_ptr(), _stream()))
        return Mat(kind, rows, cols, dst)


def mat_part(w: Mat, row_ranges, col0: int, n_cols: int) -> Mat:
    """The part of w that a tensor-parallel shard holds: row_ranges = [(first row, rows), ...] one after the other, columns
    [col0, col0 + n_cols) in whole blocks."""
    import ctypes as C

    lib = _lib.load()
    n = len(row_ranges)
    r0 = (C.c_uint32 * n)(*[int(a) for a, _ in row_ranges])
    nr = (C.c_uint32 * n)(*[int(b) for _, b in row_ranges])
    rows = sum(int(b) for _, b in row_ranges)
    dst = torch.empty(max(lib.ie_b200_mat_bytes(w.kind, rows, n_cols), 16), dtype=torch.uint8, device=w.data.device)
    check(lib.ie_b200_mat_part(w.kind, w.data.data_ptr(), w.rows, w.cols, n, r0, nr, col0, n_cols, dst.data_ptr(), _stream()))
    return Mat(w.kind, rows, n_cols, dst)


def quant_q8(x: torch.Tensor) -> torch.Tensor:
    """x: [T, n] or [n] f32 -> uint8 [T, 40 n/32] Q8 buffers."""
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    T, n = x2.shape
    nb = n // 32
    q = torch.empty((T, q8_bytes(nb)), dtype=torch.uint8, device=x.device)
    check(_lib.load().ie_b200_quant_q8(x2.data_ptr(), q.data_ptr(), nb, T, n * 4, q8_bytes(nb), _stream()))
    return q


def gemv(w: Mat, x: torch.Tensor, bias: torch.Tensor | None = None, res: torch.Tensor | None = None,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """y[T, rows] = W x (+bias) (+res). x: Q8 buffers [T, 40 nb] uint8 (f32 [T, cols] for MAT_F32)."""
    x2 = x.reshape(-1, x.shape[-1])
    T = x2.shape[0]
    y = out if out is not None else torch.empty((T, w.rows), dtype=torch.float32, device=x.device)
    xs = x2.stride(0) * x2.element_size()
    rs = 0 if res is None else res.reshape(T, -1).stride(0) * 4
    check(_lib.load().ie_b200_gemv(w.kind, w.data.data_ptr(), w.rows, w.cols, x2.data_ptr(), y.data_ptr(), _p(bias), _p(res), T, xs,
                                   w.rows * 4, rs, _stream()))
    return y


def gemm(w: Mat, x: torch.Tensor, bias: torch.Tensor | None = None, res: torch.Tensor | None = None) -> torch.Tensor:
    """The prompt-chunk form of gemv (tensor cores; equal to gemv to fp32 rounding). x: Q8 buffers [T, 40 nb] uint8."""
    x2 = x.reshape(-1, x.shape[-1])
    T = x2.shape[0]
    y = torch.empty((T, w.rows), dtype=torch.float32, device=x.device)
    rs = 0 if res is None else res.reshape(T, -1).stride(0) * 4
    check(_lib.load().ie_b200_gemm(w.kind, w.data.data_ptr(), w.rows, w.cols, x2.data_ptr(), y.data_ptr(), _p(bias), _p(res), T,
                                   x2.stride(0) * x2.element_size(), w.rows * 4, rs, _stream()))
    return y


def gemm_tc(w: Mat, x: torch.Tensor, bias: torch.Tensor | None = None, res: torch.Tensor | None = None, err: torch.Tensor | None = None) -> torch.Tensor:
    """The prompt-chunk GEMM on tcgen05 / tensor memory (equal to gemv to fp32 rounding). x: Q8 buffers [T, 40 nb] uint8."""
    lib = _lib.load()
    x2 = x.reshape(-1, x.shape[-1])
    T = x2.shape[0]
    y = torch.empty((T, w.rows), dtype=torch.float32, device=x.device)
    rs = 0 if res is None else res.reshape(T, -1).stride(0) * 4
    nbytes = lib.ie_b200_gemm_tc_scratch_bytes(w.rows, w.cols, T)
    scratch = torch.empty(nbytes + 256, dtype=torch.uint8, device=x.device)
    base = (scratch.data_ptr() + 255) // 256 * 256
    if getattr(w, "tc_exp", None) is None:
        e = ctypes.c_int(0)
        check(lib.ie_b200_mat_tc_exp(w.kind, w.data.data_ptr(), w.rows, w.cols, ctypes.byref(e), _stream()))
        w.tc_exp = e.value
    check(lib.ie_b200_gemm_tc(w.kind, w.data.data_ptr(), w.rows, w.cols, w.tc_exp, x2.data_ptr(), y.data_ptr(), _p(bias), _p(res), T,
                              x2.stride(0) * x2.element_size(), w.rows * 4, rs, base, nbytes, _p(err), _stream()))
    return y


def gemv_stream(w: Mat, xq: torch.Tensor, bias=None, res=None) -> torch.Tensor:
    """The one-token decode GEMV (same result as gemv with one row)."""
    y = torch.empty((1, w.rows), dtype=torch.float32, device=xq.device)
    check(_lib.load().ie_b200_gemv_stream(w.kind, w.data.data_ptr(), w.rows, w.cols, xq.data_ptr(), y.data_ptr(), _p(bias), _p(res), _stream()))
    return y


def norm_gemv_stream(w: Mat, x: torch.Tensor, norm_w: torch.Tensor, eps: float, bias=None, res=None):
    """y = W Q8(rmsnorm(x) * norm_w) with the norm folded into the GEMV; returns (y, xn, xq)."""
    n = w.cols
    y = torch.empty((1, w.rows), dtype=torch.float32, device=x.device)
    xn = torch.empty(n, dtype=torch.float32, device=x.device)
    xq = torch.empty(q8_bytes(n // 32), dtype=torch.uint8, device=x.device)
    check(_lib.load().ie_b200_norm_gemv_stream(w.kind, w.data.data_ptr(), w.rows, w.cols, x.data_ptr(), norm_w.data_ptr(), eps, xn.data_ptr(),
                                               xq.data_ptr(), y.data_ptr(), _p(bias), _p(res), _stream()))
    return y, xn, xq


def block_dots(w: Mat, xq: torch.Tensor) -> torch.Tensor:
    n = w.rows * w.nb * (2 if w.kind == MAT_Q6K else 1)
    d = torch.empty(n, dtype=torch.int32, device=xq.device)
    check(_lib.load().ie_b200_block_dots(w.kind, w.data.data_ptr(), w.rows, w.cols, xq.data_ptr(), d.data_ptr(), _stream()))
    return d


def embed(w: Mat, tok: torch.Tensor) -> torch.Tensor:
    T = tok.numel()
    out = torch.empty((T, w.cols), dtype=torch.float32, device=tok.device)
    check(_lib.load().ie_b200_embed(w.kind, w.data.data_ptr(), w.cols, tok.data_ptr(), out.data_ptr(), T, w.cols * 4, _stream()))
    return out


def rmsnorm(x: torch.Tensor, wt: torch.Tensor, eps: float, quant: bool = True):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    T, n = x2.shape
    y = torch.empty_like(x2)
    q = torch.empty((T, q8_bytes(n // 32)), dtype=torch.uint8, device=x.device) if quant else None
    check(_lib.load().ie_b200_rmsnorm(x2.data_ptr(), wt.data_ptr(), y.data_ptr(), n, eps, _p(q), T, n * 4, n * 4,
                                      q8_bytes(n // 32), _stream()))
    return y, q


def swiglu(gu: torch.Tensor, n: int, quant: bool = True):
    """gu: [T, 2 n] f32 ([gate | up]); gate is overwritten with silu(gate) * up."""
    T = gu.shape[0]
    q = torch.empty((T, q8_bytes(n // 32)), dtype=torch.uint8, device=gu.device) if quant else None
    check(_lib.load().ie_b200_swiglu(gu.data_ptr(), gu.data_ptr() + 4 * n, n, _p(q), T, gu.stride(0) * 4, q8_bytes(n // 32), _stream()))
    return gu[:, :n], q


def rope_kv(qkv: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
            nq: int, nkv: int, hd: int, neox: bool, kv_len: int) -> None:
    """qkv: [T, (nq + 2 nkv) hd] f32, rotated in place; kc / vc: [nkv, kv_len, hd] half or float."""
    T = qkv.shape[0]
    base = qkv.data_ptr()
    check(_lib.load().ie_b200_rope_kv(base, base + 4 * nq * hd, base + 4 * (nq + nkv) * hd, kc.data_ptr(), vc.data_ptr(), cos.data_ptr(),
                                      sin.data_ptr(), pos.data_ptr(), nq, nkv, hd, int(neox), int(kc.dtype == torch.float32), kv_len, T,
                                      qkv.stride(0) * 4, _stream()))


class AttnScratch:
    """Partials and arrival counters of the split-KV attention for one shape."""

    def __init__(self, n_head: int, hd: int, n_ctx: int, T: int, device):
        lib = _lib.load()
        self.part = torch.empty(lib.ie_b200_attn_part_bytes(n_head, hd, n_ctx, T), dtype=torch.uint8, device=device)
        self.count = torch.zeros(lib.ie_b200_attn_count_words(n_head, T), dtype=torch.int32, device=device)


def attn_decode(q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, pos: torch.Tensor, n_head: int, n_kv: int, hd: int, n_ctx: int,
                scratch: AttnScratch, quant: bool = True):
    """q: [T, >= n_head hd] f32 rows (stride taken from the tensor); returns (out [T, n_head hd], Q8 copy or None)."""
    T = q.shape[0]
    kv_len = kc.shape[1]
    out = torch.empty((T, n_head * hd), dtype=torch.float32, device=q.device)
    nbq = n_head * hd // 32
    oq = torch.empty((T, q8_bytes(nbq)), dtype=torch.uint8, device=q.device) if quant else None
    check(_lib.load().ie_b200_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), _p(oq), pos.data_ptr(), n_head, n_kv,
                                          hd, int(kc.dtype == torch.float32), kv_len, n_ctx, T, q.stride(0) * 4, n_head * hd * 4,
                                          q8_bytes(nbq), scratch.part.data_ptr(), scratch.count.data_ptr(), _stream()))
    return out, oq


def attn_decode_fused(qkv: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
                      n_head: int, n_kv: int, hd: int, neox: bool, n_ctx: int, scratch: AttnScratch, quant: bool = True):
    """One token: qkv [(n_head + 2 n_kv) hd] un-rotated; RoPE, cache store and attention in one kernel. Returns (out, Q8 copy)."""
    out = torch.empty((1, n_head * hd), dtype=torch.float32, device=qkv.device)
    nbq = n_head * hd // 32
    oq = torch.empty((1, q8_bytes(nbq)), dtype=torch.uint8, device=qkv.device) if quant else None
    base = qkv.data_ptr()
    check(_lib.load().ie_b200_attn_decode_fused(base, base + 4 * n_head * hd, base + 4 * (n_head + n_kv) * hd, kc.data_ptr(), vc.data_ptr(),
                                                cos.data_ptr(), sin.data_ptr(), out.data_ptr(), _p(oq), pos.data_ptr(), n_head, n_kv, hd, int(neox),
                                                int(kc.dtype == torch.float32), kc.shape[1], n_ctx, scratch.part.data_ptr(),
                                                scratch.count.data_ptr(), _stream()))
    return out, oq


def attn_persistent(qkv: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
                    n_head: int, n_kv: int, hd: int, neox: bool, quant: bool = True):
    """One token's RoPE + cache store + attention as the persistent step kernel runs it (half caches). `pos` must be the second
    element of an int32 tensor of at least two (the kernel addresses it as scalars[1]). Returns (out, Q8 copy, error word)."""
    lib = _lib.load()
    out = torch.empty((1, n_head * hd), dtype=torch.float32, device=qkv.device)
    nbq = n_head * hd // 32
    oq = torch.empty((1, q8_bytes(nbq)), dtype=torch.uint8, device=qkv.device) if quant else None
    scratch = torch.empty(lib.ie_b200_attn_persistent_scratch_bytes(n_head, n_kv, hd), dtype=torch.uint8, device=qkv.device)
    err = torch.zeros(4, dtype=torch.int32, device=qkv.device)
    check(lib.ie_b200_attn_persistent(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), cos.data_ptr(), sin.data_ptr(), out.data_ptr(), _p(oq),
                                      pos.data_ptr(), n_head, n_kv, hd, int(neox), kc.shape[1], scratch.data_ptr(), err.data_ptr(), _stream()))
    return out, oq, err


def attn_prefill(q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, pos: torch.Tensor, n_head: int, n_kv: int, hd: int, quant: bool = True):
    """A prompt chunk: q [T, >= n_head hd] f32 rows (rotated), half caches [n_kv, kv_len, hd] that already hold the chunk's rows;
    returns (out [T, n_head hd], Q8 copies or None)."""
    T = q.shape[0]
    out = torch.empty((T, n_head * hd), dtype=torch.float32, device=q.device)
    nbq = n_head * hd // 32
    oq = torch.empty((T, q8_bytes(nbq)), dtype=torch.uint8, device=q.device) if quant else None
    check(_lib.load().ie_b200_attn_prefill(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), _p(oq), pos.data_ptr(), n_head, n_kv, hd,
                                           kc.shape[1], T, q.stride(0) * 4, n_head * hd * 4, q8_bytes(nbq), _stream()))
    return out, oq


def topk(x: torch.Tensor, K: int):
    """x: [T, n] f32 -> (values [T, K], indices [T, K] int32): per row descending, equal values by rising index."""
    x2 = x.reshape(-1, x.shape[-1])
    T, n = x2.shape
    lib = _lib.load()
    scratch = torch.empty(lib.ie_b200_topk_scratch_bytes(n, K, T), dtype=torch.uint8, device=x.device)
    val = torch.empty((T, K), dtype=torch.float32, device=x.device)
    idx = torch.empty((T, K), dtype=torch.int32, device=x.device)
    check(lib.ie_b200_topk(x2.data_ptr(), n, K, T, x2.stride(0) * 4, val.data_ptr(), idx.data_ptr(), scratch.data_ptr(), _stream()))
    return val, idx


def argmax(x: torch.Tensor) -> torch.Tensor:
    """x: [T, n] f32 -> int32 [T, 2]: (index, float bits of the softmax probability of the maximum)."""
    x2 = x.reshape(-1, x.shape[-1])
    T, n = x2.shape
    lib = _lib.load()
    part = torch.empty(lib.ie_b200_argmax_part_bytes(T), dtype=torch.uint8, device=x.device)
    out = torch.empty((T, 2), dtype=torch.int32, device=x.device)
    check(lib.ie_b200_argmax(x2.data_ptr(), n, out.data_ptr(), T, x2.stride(0) * 4, 8, part.data_ptr(), _stream()))
    return out
