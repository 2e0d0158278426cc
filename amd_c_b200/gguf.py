"""Minimal GGUF v3 writer / reader and the seeded synthetic decoder models.

Only what the decode path needs: scalar metadata (u32, f32, string) and
tensors of type F32, Q4_0, Q4_K, Q6_K. Tensor data is aligned to 32 bytes.
The metadata keys and tensor names are the ones a llama / qwen2 GGUF carries
(general.architecture, {arch}.block_count, ..., blk.N.attn_q.weight, ...).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

from . import synth
from .synth import GGML_F32, GGML_Q4_0, GGML_Q4_K, GGML_Q6_K, GGML_Q8_0

T_U32, T_F32, T_STR = 4, 6, 8
ALIGN = 32

MAT_NAMES = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")


@dataclass
class Tensor:
    ggml_type: int
    rows: int  # ne[1] (1 for vectors)
    cols: int  # ne[0]
    data: np.ndarray  # raw bytes (uint8), any shape

    def raw(self) -> np.ndarray:
        return np.ascontiguousarray(self.data).view(np.uint8).reshape(-1)

    def f32(self) -> np.ndarray:
        assert self.ggml_type == GGML_F32
        return self.raw().view(np.float32)


@dataclass
class ModelConfig:
    arch: str = "llama"
    n_layer: int = 4
    dim: int = 256
    ffn: int = 768
    n_head: int = 8
    n_kv: int = 4
    vocab: int = 1024
    ctx: int = 512
    eps: float = 1e-5
    rope_base: float = 10000.0
    qkv_bias: bool = False
    # GGML type of each matrix family
    t_attn: int = GGML_Q4_0   # q, k, o
    t_v: int = GGML_Q4_0
    t_ffn: int = GGML_Q4_0    # gate, up
    t_down: int = GGML_Q4_0
    t_embd: int = GGML_F32
    t_out: int = GGML_F32
    tensors: dict = field(default_factory=dict, repr=False)

    @property
    def hd(self) -> int:
        return self.dim // self.n_head

    @property
    def neox(self) -> bool:
        return self.arch == "qwen2"

    def as_dict(self) -> dict:
        return dict(n_layer=self.n_layer, dim=self.dim, ffn=self.ffn, n_head=self.n_head, n_kv=self.n_kv, vocab=self.vocab, eps=self.eps,
                    rope_base=self.rope_base, neox=self.neox)


# The benchmark configurations (shapes only; weights are seeded synthetic).
def config(name: str) -> ModelConfig:
    if name == "tiny":  # 4 layers, dim 256, 8/4 heads of 32, ffn 768, vocab 1024, all Q4_0, f32 embeddings and head
        return ModelConfig()
    if name == "tiny-k":  # the same skeleton with K-quants (dims multiples of 256) and a qwen2-style bias / rope
        return ModelConfig(arch="qwen2", n_layer=2, dim=512, ffn=1536, n_head=8, n_kv=4, vocab=512, ctx=256, eps=1e-6, rope_base=1e6,
                           qkv_bias=True, t_attn=GGML_Q4_K, t_v=GGML_Q6_K, t_ffn=GGML_Q4_K, t_down=GGML_Q6_K)
    if name == "tiny-128":  # a small llama with heads of 128 (4 query / 2 KV heads): the head size of every benchmark model
        return ModelConfig(n_layer=3, dim=512, ffn=1024, n_head=4, n_kv=2, vocab=768, ctx=512, t_embd=GGML_Q4_0, t_out=GGML_Q4_0)
    if name == "tiny-kq":  # K-quants end to end (Q6_K output head, Q4_0 embedding), qwen2-style bias / rope, 16 / 8 heads of 64
        return ModelConfig(arch="qwen2", n_layer=2, dim=1024, ffn=1024, n_head=16, n_kv=8, vocab=512, ctx=256, eps=1e-6, rope_base=1e6,
                           qkv_bias=True, t_attn=GGML_Q4_K, t_v=GGML_Q6_K, t_ffn=GGML_Q4_K, t_down=GGML_Q6_K, t_embd=GGML_Q4_0, t_out=GGML_Q6_K)
    if name == "tiny-q8":  # every matrix Q8_0 (what the reference keeps as its MAT_Q8 kind), f32 embedding, Q8_0 output head
        return ModelConfig(n_layer=3, dim=256, ffn=768, n_head=8, n_kv=4, vocab=1024, ctx=512, t_attn=GGML_Q8_0, t_v=GGML_Q8_0, t_ffn=GGML_Q8_0,
                           t_down=GGML_Q8_0, t_out=GGML_Q8_0)
    if name == "tiny-tp":  # all Q4_0, 16 / 8 heads of 64: shards over 2, 4 or 8 ranks
        return ModelConfig(n_layer=3, dim=1024, ffn=2048, n_head=16, n_kv=8, vocab=1024, ctx=512, t_embd=GGML_Q4_0, t_out=GGML_Q4_0)
    if name == "llama3-8b":
        return ModelConfig(n_layer=32, dim=4096, ffn=14336, n_head=32, n_kv=8, vocab=128256, ctx=8192, rope_base=500000.0,
                           t_embd=GGML_Q4_0, t_out=GGML_Q4_0)
    if name == "llama3-8b-f32head":
        return ModelConfig(n_layer=32, dim=4096, ffn=14336, n_head=32, n_kv=8, vocab=128256, ctx=8192, rope_base=500000.0)
    if name == "qwen2-7b-q4km":
        return ModelConfig(arch="qwen2", n_layer=28, dim=3584, ffn=18944, n_head=28, n_kv=4, vocab=152064, ctx=8192, eps=1e-6, rope_base=1e6,
                           qkv_bias=True, t_attn=GGML_Q4_K, t_v=GGML_Q6_K, t_ffn=GGML_Q4_K, t_down=GGML_Q6_K, t_embd=GGML_Q4_0,
                           t_out=GGML_Q6_K)
    if name == "dense-27b-q4km":
        return ModelConfig(arch="qwen2", n_layer=64, dim=5120, ffn=17408, n_head=40, n_kv=8, vocab=152064, ctx=33024, eps=1e-6, rope_base=1e6,
                           t_attn=GGML_Q4_K, t_v=GGML_Q6_K, t_ffn=GGML_Q4_K, t_down=GGML_Q6_K, t_embd=GGML_Q4_0, t_out=GGML_Q6_K)
    raise KeyError(name)


def tensor_plan(cfg: ModelConfig):
    """(name, ggml_type, rows, cols) of every tensor, in file order."""
    kvd = cfg.n_kv * cfg.hd
    plan = [("token_embd.weight", cfg.t_embd, cfg.vocab, cfg.dim)]
    for l in range(cfg.n_layer):
        p = f"blk.{l}."
        plan.append((p + "attn_norm.weight", GGML_F32, 1, cfg.dim))
        plan.append((p + "attn_q.weight", cfg.t_attn, cfg.dim, cfg.dim))
        plan.append((p + "attn_k.weight", cfg.t_attn, kvd, cfg.dim))
        plan.append((p + "attn_v.weight", cfg.t_v, kvd, cfg.dim))
        if cfg.qkv_bias:
            plan.append((p + "attn_q.bias", GGML_F32, 1, cfg.dim))
            plan.append((p + "attn_k.bias", GGML_F32, 1, kvd))
            plan.append((p + "attn_v.bias", GGML_F32, 1, kvd))
        plan.append((p + "attn_output.weight", cfg.t_attn, cfg.dim, cfg.dim))
        plan.append((p + "ffn_norm.weight", GGML_F32, 1, cfg.dim))
        plan.append((p + "ffn_gate.weight", cfg.t_ffn, cfg.ffn, cfg.dim))
        plan.append((p + "ffn_up.weight", cfg.t_ffn, cfg.ffn, cfg.dim))
        plan.append((p + "ffn_down.weight", cfg.t_down, cfg.dim, cfg.ffn))
    plan.append(("output_norm.weight", GGML_F32, 1, cfg.dim))
    plan.append(("output.weight", cfg.t_out, cfg.vocab, cfg.dim))
    return plan


def is_matrix(name: str) -> bool:
    return name in ("token_embd.weight", "output.weight") or (name.endswith(".weight") and name.split(".")[-2] in MAT_NAMES)


def make_model(cfg: ModelConfig, seed: int = 0, sigma: float = 0.02) -> ModelConfig:
    """Fill cfg.tensors with seeded synthetic weights (numpy; for the small configurations)."""
    rng = np.random.default_rng(seed)
    cfg.tensors = {}
    for name, typ, rows, cols in tensor_plan(cfg):
        if not is_matrix(name):
            if name.endswith("norm.weight"):
                v = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
            else:
                v = (sigma * rng.standard_normal(cols)).astype(np.float32)
            cfg.tensors[name] = Tensor(GGML_F32, 1, cols, v.view(np.uint8))
        else:
            cfg.tensors[name] = Tensor(typ, rows, cols, synth.make_gguf_bytes(typ, rng, rows, cols, sigma))
    return cfg


# ---------------------------------------------------------------- file format

def _s(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, cfg: ModelConfig) -> None:
    a = cfg.arch
    kvs = [
        ("general.architecture", T_STR, a), ("general.name", T_STR, "synthetic-" + a), ("general.alignment", T_U32, ALIGN),
        (a + ".block_count", T_U32, cfg.n_layer), (a + ".context_length", T_U32, cfg.ctx), (a + ".embedding_length", T_U32, cfg.dim),
        (a + ".feed_forward_length", T_U32, cfg.ffn), (a + ".attention.head_count", T_U32, cfg.n_head),
        (a + ".attention.head_count_kv", T_U32, cfg.n_kv), (a + ".attention.layer_norm_rms_epsilon", T_F32, cfg.eps),
        (a + ".rope.freq_base", T_F32, cfg.rope_base),
    ]
    out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(cfg.tensors), len(kvs)))
    for k, t, v in kvs:
        out += _s(k) + struct.pack("<I", t)
        out += _s(v) if t == T_STR else struct.pack("<I" if t == T_U32 else "<f", v)
    off = 0
    for name, t in cfg.tensors.items():
        ne = [t.cols] if not is_matrix(name) else [t.cols, t.rows]
        out += _s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", t.ggml_type, off)
        off += (t.raw().size + ALIGN - 1) // ALIGN * ALIGN
    out += b"\0" * ((-len(out)) % ALIGN)
    with open(path, "wb") as f:
        f.write(out)
        for t in cfg.tensors.values():
            raw = t.raw()
            f.write(raw.tobytes())
            f.write(b"\0" * ((-raw.size) % ALIGN))


def read_gguf(path) -> ModelConfig:
    buf = np.fromfile(path, dtype=np.uint8)
    mv = memoryview(buf)
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, mv, pos)
        pos += struct.calcsize(fmt)
        return v[0] if len(v) == 1 else v

    def take_str():
        nonlocal pos
        n = take("<Q")
        s = bytes(mv[pos:pos + n]).decode("utf-8")
        pos += n
        return s

    if bytes(mv[:4]) != b"GGUF":
        raise ValueError("not a GGUF file")
    pos = 4
    version, n_t, n_kv = take("<IQQ")
    if version != 3:
        raise ValueError(f"GGUF version {version}")
    meta = {}
    for _ in range(n_kv):
        k = take_str()
        t = take("<I")
        if t == T_STR:
            meta[k] = take_str()
        elif t == T_U32:
            meta[k] = take("<I")
        elif t == T_F32:
            meta[k] = take("<f")
        else:
            raise ValueError(f"metadata type {t} of {k} unsupported by this reader")
    infos = []
    for _ in range(n_t):
        name = take_str()
        nd = take("<I")
        ne = [take("<Q") for _ in range(nd)]
        typ, off = take("<IQ")
        infos.append((name, ne, typ, off))
    align = meta.get("general.alignment", ALIGN)
    base = (pos + align - 1) // align * align
    a = meta["general.architecture"]
    cfg = ModelConfig(arch=a, n_layer=meta[a + ".block_count"], dim=meta[a + ".embedding_length"], ffn=meta[a + ".feed_forward_length"],
                      n_head=meta[a + ".attention.head_count"], n_kv=meta[a + ".attention.head_count_kv"], ctx=meta[a + ".context_length"],
                      eps=meta.get(a + ".attention.layer_norm_rms_epsilon", 1e-5), rope_base=meta.get(a + ".rope.freq_base", 10000.0))
    for name, ne, typ, off in infos:
        cols, rows = ne[0], (ne[1] if len(ne) > 1 else 1)
        n = synth.gguf_nbytes(typ, rows, cols)
        cfg.tensors[name] = Tensor(typ, rows, cols, buf[base + off: base + off + n])
    cfg.vocab = cfg.tensors["token_embd.weight"].rows
    cfg.qkv_bias = "blk.0.attn_q.bias" in cfg.tensors
    t = cfg.tensors
    cfg.t_attn, cfg.t_v = t["blk.0.attn_q.weight"].ggml_type, t["blk.0.attn_v.weight"].ggml_type
    cfg.t_ffn, cfg.t_down = t["blk.0.ffn_gate.weight"].ggml_type, t["blk.0.ffn_down.weight"].ggml_type
    cfg.t_embd = t["token_embd.weight"].ggml_type
    cfg.t_out = t["output.weight"].ggml_type if "output.weight" in t else cfg.t_embd
    return cfg


def make_model_device(cfg: ModelConfig, seed: int = 0, sigma: float = 0.02, device="cuda"):
    """As make_model, for the large configurations: matrices are generated on the GPU (torch generator, same
    block definition) and returned as name -> (ggml_type, rows, cols, uint8 CUDA tensor); the small float
    vectors go to cfg.tensors as numpy. Pass the dict as Backend(device_tensors=...)."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)
    rng = np.random.default_rng(seed)
    cfg.tensors, dev = {}, {}
    for name, typ, rows, cols in tensor_plan(cfg):
        if not is_matrix(name):
            if name.endswith("norm.weight"):
                v = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
            else:
                v = (sigma * rng.standard_normal(cols)).astype(np.float32)
            cfg.tensors[name] = Tensor(GGML_F32, 1, cols, v.view(np.uint8))
        elif typ == GGML_Q4_0:
            dev[name] = (typ, rows, cols, synth.q4_0_normal_torch(gen, rows, cols, sigma, device=device).reshape(-1))
        elif typ == GGML_F32:
            dev[name] = (typ, rows, cols, (torch.randn((rows, cols), generator=gen, device=device) * sigma).view(torch.uint8).reshape(-1))
        else:
            dev[name] = (typ, rows, cols, synth.k_random_torch(typ, gen, rows, cols, sigma, device=device).reshape(-1))
    return dev
