"""Generate tests/golden/*.npz from the reference's own CPU code.

Run where the reference tree is present (oracle/_ref/libie_ref.so gets built
from it): python tests/golden/make_golden.py
The fixtures hold seeded inputs and the reference's outputs, so that the
restatement (oracle/ie_oracle.c) and the CUDA kernels can be checked on
machines that do not have the reference tree.

  kernels.npz  Q8 quantiser outputs; GEMV outputs for Q4_0 / Q4_K / Q6_K / Q8_0 on
               the shape list of the reference's tests/kernel_test.c plus
               K-quant shapes; the reference's repacked arrays' checksums
  tiny.npz     the tiny 4-layer Q4_0 llama (seed 0): greedy ids of 64 tokens
               from prompt 1,2,3 at context 512, logits of the first 8 steps,
               per-layer residual outputs of steps 0..3
  tiny_k.npz   the K-quant qwen2-style tiny model: 24 greedy ids, logits of 4 steps
  tiny_q8.npz  the tiny llama with every matrix Q8_0: 24 greedy ids, logits of 4 steps
"""
from __future__ import annotations

import hashlib
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from amd_c_b200 import gguf, synth  # noqa: E402
from oracle.oracle import Ref, RefEngine  # noqa: E402

OUT = Path(__file__).resolve().parent
Q4_SHAPES = [(1, 1), (7, 3), (9, 11), (8, 32), (13, 33), (17, 36), (5, 64), (3, 100), (2, 511)]  # (rows, blocks) of kernel_test.c
K_SHAPES = [(3, 8), (9, 16), (8, 40), (5, 112), (2, 448)]


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def kernels(ref: Ref) -> None:
    rng = np.random.default_rng(1234)
    out = {}
    x = rng.standard_normal(32 * 24).astype(np.float32)
    x[32:64] = 0.0  # a zero block: d = 0, q = 0
    x[64] = 127.5 * 0.01
    x[65:96] = 0.01  # ties at .5 after division
    out["quant_x"], out["quant_q"] = x, ref.quant_q8(x)
    # (Q8_0 last: the draws of the kinds before it, and so their fixtures, stay what they were)
    for typ, shapes, tag in ((synth.GGML_Q4_0, Q4_SHAPES, "q4_0"), (synth.GGML_Q4_K, K_SHAPES, "q4_k"), (synth.GGML_Q6_K, K_SHAPES, "q6_k"),
                             (synth.GGML_Q8_0, Q4_SHAPES, "q8_0")):
        for rows, nb in shapes:
            cols = nb * 32
            raw = synth.make_gguf_bytes(typ, rng, rows, cols)
            xs = (rng.standard_normal(cols) * np.where(np.arange(cols) % 7 == 0, 3.0, 1.0)).astype(np.float32)
            xq = ref.quant_q8(xs)
            m = ref.mat(typ, raw, rows, cols)
            qw, qs = m.arrays()
            key = f"{tag}_{rows}x{nb}"
            out[key + "_raw"], out[key + "_x"], out[key + "_y"] = raw.reshape(-1), xs, m.gemv(xq)
            out[key + "_sha"] = np.frombuffer((sha(qw) + sha(qs)).encode(), dtype=np.uint8)
            m.free()
    np.savez_compressed(OUT / "kernels.npz", **out)


def model(ref: Ref, name: str, seed: int, n_ctx: int, n_gen: int, n_logits: int, n_trace: int, fname: str) -> None:
    cfg = gguf.make_model(gguf.config(name), seed=seed)
    with tempfile.TemporaryDirectory() as td:
        path = Path(td) / "m.gguf"
        gguf.write_gguf(path, cfg)
        file_sha = hashlib.sha256(path.read_bytes()).hexdigest()
        eng = RefEngine(ref, str(path), n_ctx)
        prompt = [1, 2, 3]
        ids, logits, traces = list(prompt), [], []
        tok = prompt[0]
        for pos in range(len(prompt) + n_gen - 1):
            if pos < n_trace:
                traces.append(eng.layer_outputs(tok, pos))
            nxt, lg, _ = eng.step(tok, pos)
            if pos < n_logits:
                logits.append(lg)
            if pos + 1 < len(prompt):
                tok = prompt[pos + 1]
            else:
                tok = nxt
                ids.append(nxt)
        wb = eng.weight_bytes_per_token()
        eng.close()
    np.savez_compressed(OUT / fname, ids=np.array(ids, np.uint32), logits=np.stack(logits), traces=np.stack(traces) if traces else np.zeros(0),
                        gguf_sha=np.frombuffer(file_sha.encode(), dtype=np.uint8), seed=seed, n_ctx=n_ctx, weight_bytes_per_token=wb)


if __name__ == "__main__":
    r = Ref()
    kernels(r)
    model(r, "tiny", 0, 512, 64, 8, 4, "tiny.npz")
    model(r, "tiny-k", 0, 256, 24, 4, 2, "tiny_k.npz")
    model(r, "tiny-q8", 0, 256, 24, 4, 2, "tiny_q8.npz")
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)
