"""Small stand-alone cases of the hot kernels, sized for a profiler: few launches, a few GB on the device at most,
inputs larger than L2 where DRAM figures matter.

  python -m amd_c_b200.cases gemv [rows cols [q4_0|q4_k|q6_k [launches]]]   decode GEMV on rotating copies of one matrix
  python -m amd_c_b200.cases gemm [rows cols T [q4_0|q4_k|q6_k]]             prompt-chunk GEMM
  python -m amd_c_b200.cases attn [positions [launches]]                     decode attention, Llama-3-8B heads, f16 cache
  python -m amd_c_b200.cases step [config [position [steps]]]               whole decode steps as plain launches (no graph)

Each prints the CUDA-event time per launch; under ncu select the kernel with -k regex:<name>.
"""
from __future__ import annotations

import sys

import numpy as np
import torch

from . import gguf, synth
from . import kernels as K
from .backend import Backend

KINDS = {"q4_0": synth.GGML_Q4_0, "q4_k": synth.GGML_Q4_K, "q6_k": synth.GGML_Q6_K}


def _matrix(typ: int, rows: int, cols: int, gen, dev) -> K.Mat:
    raw = synth.q4_0_normal_torch(gen, rows, cols, device=dev) if typ == synth.GGML_Q4_0 else synth.k_random_torch(typ, gen, rows, cols, device=dev)
    return K.Mat.from_gguf(typ, raw.reshape(-1), rows, cols)


def _timed(fn, n: int) -> float:
    """n launches; the time per launch is taken over the last n - 1 (the first pays the one-time set-up)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn(0)
    e0.record()
    for i in range(1, n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / max(1, n - 1)


def case_gemv(rows=14336, cols=4096, kind="q4_0", launches=12):
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(0)
    m = _matrix(KINDS[kind], int(rows), int(cols), gen, dev)
    ncopy = max(2, min(16, int(300e6 // m.data.numel()) + 1))  # more than the 126 MB L2 between two uses of a copy
    copies = [K.Mat(m.kind, m.rows, m.cols, m.data.clone()) for _ in range(ncopy)]
    xq = K.quant_q8(torch.randn(1, int(cols), device=dev, generator=gen))
    us = _timed(lambda i: K.gemv_stream(copies[i % ncopy], xq), int(launches))
    print(f"gemv {kind} {rows}x{cols}: {us:.2f} us per launch (plain launches, {ncopy} copies), {m.algorithmic_bytes / us / 1e3:.0f} GB/s")


def case_gemm(rows=28672, cols=4096, T=256, kind="q4_0"):
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(0)
    m = _matrix(KINDS[kind], int(rows), int(cols), gen, dev)
    xq = K.quant_q8(torch.randn(int(T), int(cols), device=dev, generator=gen))
    us = _timed(lambda i: K.gemm(m, xq), 4)
    print(f"gemm {kind} {rows}x{cols} T={T}: {us:.1f} us per launch, {2.0 * int(rows) * int(cols) * int(T) / us / 1e6:.1f} TFLOP/s")


def case_attn(positions=4096, launches=6):
    dev = torch.device("cuda:0")
    n_head, n_kv, hd, n_ctx = 32, 8, 128, int(positions) + 8
    gen = torch.Generator(device=dev).manual_seed(0)
    nl = max(2, int(300e6 // (2 * n_kv * n_ctx * hd * 2)) + 1)  # layers' worth of caches, so that each launch reads cold rows
    kc = [(torch.randn(n_kv, n_ctx, hd, device=dev, generator=gen) * 0.5).half() for _ in range(nl)]
    vc = [(torch.randn(n_kv, n_ctx, hd, device=dev, generator=gen) * 0.5).half() for _ in range(nl)]
    cos, sin = torch.ones(n_ctx, hd // 2, device=dev), torch.zeros(n_ctx, hd // 2, device=dev)
    qkv = torch.randn((n_head + 2 * n_kv) * hd, device=dev, generator=gen)
    pos = torch.tensor([int(positions)], dtype=torch.int32, device=dev)
    sc = K.AttnScratch(n_head, hd, n_ctx, 1, dev)
    us = _timed(lambda i: K.attn_decode_fused(qkv, kc[i % nl], vc[i % nl], cos, sin, pos, n_head, n_kv, hd, False, n_ctx, sc), int(launches))
    kv_bytes = 2 * (int(positions) + 1) * n_kv * hd * 2
    print(f"attn decode {positions} positions: {us:.2f} us per launch, {kv_bytes / us / 1e3:.0f} GB/s of K/V")


def case_step(config="llama3-8b", position=200, steps=3):
    dev = torch.device("cuda:0")
    cfg = gguf.config(config)
    tensors = gguf.make_model_device(cfg, seed=0)
    b = Backend(cfg, int(position) + int(steps) + 8, T=1, device_tensors=tensors, device=dev)
    del tensors
    torch.cuda.empty_cache()
    tok = 1
    for i in range(int(steps)):
        b.run_ops(tok, int(position) + i, len(b.ops))
    print(f"{config}: {steps} decode steps as plain launches at position {position}, {b.launches_per_step} launches per step")
    b.close()


def main(argv):
    cases = {"gemv": case_gemv, "gemm": case_gemm, "attn": case_attn, "step": case_step}
    if not argv or argv[0] not in cases:
        sys.exit(__doc__)
    cases[argv[0]](*argv[1:])


if __name__ == "__main__":
    main(sys.argv[1:])
