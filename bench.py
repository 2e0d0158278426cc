#!/usr/bin/env python
"""Benchmark of the decode hot path: Llama-3-8B-shaped Q4_0 greedy decode, batch 1.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one decode token (one pass of the op list over the weights). One JSON
line goes to stdout (rank 0):
  value     decode tokens/s with everything resident on the device: the step
            graph replayed K times, the argmax fed back on the device
  e2e       the same through backend.step(): token id and position from host
            memory every step, argmax read back every step
  roofline  the GEMV kernels of the step (the dominant kernel) alone, timed
            with CUDA events on their stream: algorithmic weight bytes / time
            against the measured HBM copy bandwidth; gemv_sweep: the stand-alone
            GEMV at the Llama-3-8B shapes
  attention, prefill_gemm, qwen2_7b_q4km  the other kernels and the prompt path
            (one GPU only)
  cpu_baseline  the reference's own CPU GEMV (oracle/_ref, built from its
            sources) or the oracle port, on a bounded sample, 1 core
Weights are seeded synthetic (no network, no checkpoint): N(0, 0.02) quantised
to Q4_0 as the benchmark definition says; the prompt is 128 seeded uniform ids.
With --gpus N > 1 (under torchrun) the model is sharded tensor-parallel.
--impl reference times the reference CPU implementation instead (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC, UNIT = "decode_tokens_per_s", "tokens/s"
PROMPT_LEN = 128


def measured_peaks() -> tuple[float, str]:
    """HBM GB/s to hold achieved bandwidth against: the driver-measured copy bandwidth, else the documented fallback."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path = gpu_index, None, None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.idx)],
                                         stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path:
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])), mx.append(float(c[2]))
            except ValueError:
                continue
            for n, v in zip(names, c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------ CPU side

def layer_sample_bytes(cfg) -> tuple[int, int]:
    """(algorithmic weight bytes of one layer's GEMVs, of the whole step) at 18 B per Q4_0 block."""
    kvd = cfg.n_kv * cfg.hd
    layer = (cfg.dim * cfg.dim * 2 + 2 * kvd * cfg.dim + 3 * cfg.ffn * cfg.dim) // 32 * 18
    head = cfg.vocab * cfg.dim // 32 * 18
    return layer, layer * cfg.n_layer + head


def cpu_layer_sample(cfg, seed: int = 0):
    """One layer's seven matrices (seeded, same block definition) as the CPU implementation wants them, and a Q8
    activation for each input width. Returns (callable that runs the seven GEMVs once, kind, cores)."""
    import numpy as np

    from amd_c_b200 import synth
    from oracle.oracle import Oracle, Ref

    rng = np.random.default_rng(seed)
    kvd = cfg.n_kv * cfg.hd
    shapes = [(cfg.dim, cfg.dim), (kvd, cfg.dim), (kvd, cfg.dim), (cfg.dim, cfg.dim), (cfg.ffn, cfg.dim), (cfg.ffn, cfg.dim), (cfg.dim, cfg.ffn)]
    ora = Oracle()
    xq = {c: ora.quant_q8(rng.standard_normal(c).astype(np.float32)) for c in {s[1] for s in shapes}}
    if Ref.available():
        ref = Ref()
        mats = [ref.mat(synth.GGML_Q4_0, synth.q4_0_normal(rng, r, c), r, c) for r, c in shapes]

        def run():
            for m in mats:
                m.gemv(xq[m.cols])
        return run, "reference", 1
    packed = []
    for r, c in shapes:
        kind, qw, qs = ora.repack(synth.GGML_Q4_0, synth.q4_0_normal(rng, r, c), r, c)
        packed.append((kind, qw, qs, r, c))

    def run():
        for kind, qw, qs, r, c in packed:
            ora.gemv(kind, qw, qs, r, c, xq[c])
    return run, "port", 1


def cpu_baseline(cfg, budget_s: float = 12.0) -> dict:
    """The reference CPU GEMV on one of the n_layer layers, repeated for about budget_s seconds; tokens/s
    extrapolated by weight bytes to the whole step (the GEMVs are 99 % of a CPU step)."""
    run, kind, cores = cpu_layer_sample(cfg)
    layer_b, step_b = layer_sample_bytes(cfg)
    run()
    t0, reps = time.perf_counter(), 0
    while reps < 3 or time.perf_counter() - t0 < budget_s:
        run()
        reps += 1
    per = (time.perf_counter() - t0) / reps
    return {"value": 1.0 / (per * step_b / layer_b), "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"GEMV-only sample: the 7 Q4_0 GEMVs of 1 of {cfg.n_layer} layers ({layer_b / 1e6:.1f} MB of weights) through the reference's "
                      f"cpu_gemv_q4, {reps} repetitions, extrapolated by weight bytes to the {step_b / 1e9:.3f} GB of one token (attention, norms "
                      f"and the embedding row, about 1 % of a CPU step, are not in it)", "gb_per_s": layer_b / per / 1e9}


def run_reference_arm(args, cfg, rank: int) -> None:
    """--impl reference: the reference's single-threaded CPU backend. One step = one layer's GEMVs (a bounded
    sample of a token); tokens/s extrapolated by weight bytes. Rank 0 alone works."""
    if rank != 0:
        return
    run, kind, cores = cpu_layer_sample(cfg)
    layer_b, step_b = layer_sample_bytes(cfg)
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    per = (time.perf_counter() - t0) / args.steps
    v = 1.0 / (per * step_b / layer_b)
    sample = (f"GEMV-only sample: each step = the 7 Q4_0 GEMVs of 1 of {cfg.n_layer} layers through the reference's cpu_gemv_q4 "
              f"({layer_b / 1e6:.1f} MB of weights); tokens/s extrapolated by weight bytes to one token ({step_b / 1e9:.3f} GB)")
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": 1e3 / v, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                      "dtype": "int8 dot4 + f32 accumulate", "data": "synthetic", "config": workload_config(cfg, args.gpus),
                      "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
                      "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}), flush=True)


def workload_config(cfg, n_gpus: int) -> dict:
    return {"workload": "Llama-3-8B-shaped random-init Q4_0 greedy decode, batch 1 (32 layers, d_model 4096, 32/8 heads of 128, FFN 14336, "
                        "vocab 128256, Q4_0 embedding and output head, f16 KV cache), 128-token seeded prompt",
            "prompt_len": PROMPT_LEN, "parallelism": f"tp{n_gpus}", "l2": "every step streams 4.2 GB of weights, far more than the 126 MB L2; no flush needed"}


# ------------------------------------------------------------------ GPU side

def build_backend(cfg, n_ctx: int, tp: int, rank: int, device, step_mode: str | None = None):
    import torch

    from amd_c_b200 import gguf
    from amd_c_b200.backend import Backend

    dev_tensors = gguf.make_model_device(cfg, seed=0, device=device)
    b = Backend(cfg, n_ctx, T=1, device_tensors=dev_tensors, tp=tp, rank=rank, device=device, step_mode=step_mode)
    del dev_tensors
    torch.cuda.empty_cache()
    return b


def time_gemvs(b, reps: int = 20, repeats: int = 5, mask: int | None = None) -> dict:
    """The GEMV kernels of one step alone, in op-list order on the real matrices (a chain of dependent launches, as
    in the step), captured into a graph and timed with CUDA events on the capturing stream. Every pass streams all
    weights (4.2 GB), so nothing is served from L2."""
    import torch

    from amd_c_b200 import _lib
    from amd_c_b200.backend import OP_GEMV

    lib = _lib.load()
    if mask is None:
        mask = 1 << OP_GEMV
    s = torch.cuda.Stream(device=b.device)
    with torch.cuda.device(b.device), torch.cuda.stream(s):
        before = lib.ie_b200_launch_count()
        b.enqueue_kinds(0, len(b.ops), mask, s.cuda_stream)
        launches = lib.ie_b200_launch_count() - before
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            b.enqueue_kinds(0, len(b.ops), mask, s.cuda_stream)
        for _ in range(3):
            g.replay()
        s.synchronize()
        times = []
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            for _ in range(reps):
                g.replay()
            e1.record(s)
            s.synchronize()
            times.append(e0.elapsed_time(e1) / reps)
    return {"ms_per_pass": statistics.median(times), "ms_per_pass_min": min(times), "repeats": repeats, "launches": int(launches),
            "bytes": b.weight_bytes_per_token}


# DRAM bytes (read + written) per algorithmic byte of the decode GEMV: what ncu's dram__bytes_read.sum + dram__bytes_write.sum
# gave for one launch of gemv_direct_kernel on a 14336 x 4096 Q4_0 matrix (33.030 MB of blocks). A profiler figure cannot be taken
# inside a benchmark run; the timing beside it is live.
NCU_TRAFFIC_RATIO = 33.095 / 33.030
SWEEP_SHAPES = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]
OTHER_KIND_SHAPES = [("q4_k", 37888, 3584), ("q6_k", 3584, 18944), ("q8_0", 14336, 4096)]  # the other weight kinds, one large shape each


def time_gemv_sweep(device, peak: float) -> list[dict]:
    """The stand-alone Q4_0 x Q8 GEMV at the Llama-3-8B shapes (and one large shape of each other weight kind): seeded weights,
    >= 1 GB of rotated copies per shape (nothing is served from L2), 20 warm-up + 200 timed launches in one graph between two
    CUDA events."""
    import torch

    from amd_c_b200 import kernels as K
    from amd_c_b200 import synth

    gen = torch.Generator(device=device).manual_seed(0)
    out = []
    s = torch.cuda.Stream(device=device)
    for kind, rows, cols in [("q4_0", r, c) for r, c in SWEEP_SHAPES] + OTHER_KIND_SHAPES:
        typ = {"q4_0": synth.GGML_Q4_0, "q8_0": synth.GGML_Q8_0, "q4_k": synth.GGML_Q4_K, "q6_k": synth.GGML_Q6_K}[kind]
        raw = (synth.q4_0_normal_torch(gen, rows, cols, device=device) if kind == "q4_0" else
               synth.q8_0_normal_torch(gen, rows, cols, device=device) if kind == "q8_0" else synth.k_random_torch(typ, gen, rows, cols, device=device))
        m = K.Mat.from_gguf(typ, raw.reshape(-1), rows, cols)
        del raw
        ncopy = max(4, min(64, int(1.2e9 // m.data.numel())))
        copies = [K.Mat(m.kind, rows, cols, m.data.clone()) for _ in range(ncopy)]
        xq = K.quant_q8(torch.randn(1, cols, device=device, generator=gen))
        n = 200
        with torch.cuda.stream(s):
            for i in range(20):
                K.gemv_stream(copies[i % ncopy], xq)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for i in range(n):
                    K.gemv_stream(copies[i % ncopy], xq)
            g.replay()
            s.synchronize()
            reps = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(s)
                g.replay()
                e1.record(s)
                s.synchronize()
                reps.append(e0.elapsed_time(e1) * 1e3 / n)
        us, us_min = statistics.median(reps), min(reps)
        gbs = m.algorithmic_bytes / us / 1e3
        out.append({"kind": kind, "shape": f"{rows}x{cols}", "us": round(us, 2), "us_min": round(us_min, 2), "GB/s": round(gbs, 1), "frac": round(gbs / peak, 3),
                    "frac_of_nominal_8000": round(gbs / 8000.0, 3), "copies": ncopy, "repeats": 5})
        del copies, m, g
        torch.cuda.empty_cache()
    return out


def time_attention(device, peak: float, lengths=(256, 4096, 32768), n_kv: int = 8) -> list[dict]:
    """The decode attention kernel alone (32 query / 8 KV heads of 128, f16 cache, RoPE + KV store fused) at short and
    long contexts: a graph of 40 launches over rotating caches larger than L2, CUDA events on the capturing stream.
    Algorithmic bytes: 2 x (positions + 1) x n_kv x hd x 2 B."""
    import torch

    from amd_c_b200 import kernels as K

    n_head, hd = 32, 128
    out = []
    for positions in lengths:
        n_ctx = positions + 8
        gen = torch.Generator(device=device).manual_seed(positions)
        nl = max(2, int(300e6 // (2 * n_kv * n_ctx * hd * 2)) + 1)
        kc = [(torch.randn(n_kv, n_ctx, hd, device=device, generator=gen) * 0.5).half() for _ in range(nl)]
        vc = [(torch.randn(n_kv, n_ctx, hd, device=device, generator=gen) * 0.5).half() for _ in range(nl)]
        cos, sin = torch.ones(n_ctx, hd // 2, device=device), torch.zeros(n_ctx, hd // 2, device=device)
        qkv = torch.randn((n_head + 2 * n_kv) * hd, device=device, generator=gen)
        pos = torch.tensor([positions], dtype=torch.int32, device=device)
        sc = K.AttnScratch(n_head, hd, n_ctx, 1, device)
        s = torch.cuda.Stream(device=device)
        n = 40

        def launch(i):
            K.attn_decode_fused(qkv, kc[i % nl], vc[i % nl], cos, sin, pos, n_head, n_kv, hd, False, n_ctx, sc)

        with torch.cuda.stream(s):
            for i in range(3):
                launch(i)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for i in range(n):
                    launch(i)
            g.replay()
            s.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            g.replay()
            e1.record(s)
            s.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / n
        gbs = 2.0 * (positions + 1) * n_kv * hd * 2 / us / 1e3
        out.append({"positions": positions, "us": round(us, 2), "GB/s": round(gbs, 1), "frac": round(gbs / peak, 3)})
        del kc, vc, g
        torch.cuda.empty_cache()
    return out


def time_prefill_gemm(device) -> dict:
    """The prompt-chunk GEMM on the Qwen2-7B Q4_K_M FFN shapes, one chunk of 256 tokens, both kernels: the tcgen05 one (f16 pairs,
    fp32 accumulation in tensor memory; the default) and the int8 mma.sync one (block dots + fp32 scaling on the CUDA cores).
    Reported as 2 * rows * cols * T / time (the tcgen05 kernel issues three MMAs per product term pair, so its tensor pipe does 3x that)."""
    import torch

    from amd_c_b200 import kernels as K
    from amd_c_b200 import synth

    gen = torch.Generator(device=device).manual_seed(3)
    out = {}
    for name, typ, rows, cols in (("q4_k 37888x3584", synth.GGML_Q4_K, 37888, 3584), ("q6_k 3584x18944", synth.GGML_Q6_K, 3584, 18944)):
        raw = synth.k_random_torch(typ, gen, rows, cols, device=device)
        m = K.Mat.from_gguf(typ, raw.reshape(-1), rows, cols)
        xq = K.quant_q8(torch.randn(256, cols, device=device, generator=gen))
        out[name] = {"T": 256}
        for tag, fn in (("tcgen05", K.gemm_tc), ("mma_sync", K.gemm)):
            for _ in range(3):
                fn(m, xq)
            torch.cuda.synchronize(device)
            reps = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    fn(m, xq)
                e1.record()
                torch.cuda.synchronize(device)
                reps.append(e0.elapsed_time(e1) / 5)
            ms = statistics.median(reps)
            out[name][tag] = {"us": round(ms * 1e3, 1), "us_min": round(min(reps) * 1e3, 1), "TFLOP/s": round(2.0 * rows * cols * 256 / ms / 1e9, 1)}
        del m, raw
        torch.cuda.empty_cache()
    return out


def time_qwen2_prefill(device) -> dict:
    """The Qwen2-7B-shaped Q4_K_M model (Q4_K attention / FFN, Q6_K for V and down, QKV bias): 4096 seeded uniform prompt
    ids in chunks of 256 through backend.run (tensor-core GEMM + chunk attention), then 128 greedy tokens on the device."""
    import numpy as np
    import torch

    from amd_c_b200 import gguf
    from amd_c_b200.backend import Backend, prefill

    cfg = gguf.config("qwen2-7b-q4km")
    tensors = gguf.make_model_device(cfg, seed=0)
    b = Backend(cfg, 4096 + 136, T=256, device_tensors=tensors, device=device)
    del tensors
    torch.cuda.empty_cache()
    prompt = np.random.default_rng(2).integers(0, cfg.vocab, 4096)
    prefill(b, prompt[:512], 256)  # warm-up: two chunks
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    tok = prefill(b, prompt, 256)
    torch.cuda.synchronize(device)
    dt = time.perf_counter() - t0
    out, ms = b.decode(tok, 4096, 128)
    res = {"workload": "Qwen2-7B-shaped random-init Q4_K_M, 28 layers, 4096-token prompt in chunks of 256, then 128 greedy tokens",
           "prefill_tokens_per_s": 4096 / dt, "prefill_ms_per_chunk": dt * 1e3 / 16, "decode_tokens_per_s": 128 / (ms * 1e-3),
           "decode_ms_per_step": ms / 128, "weight_gb_per_token": b.weight_bytes_per_token / 1e9}
    b.close()
    torch.cuda.empty_cache()
    return res


def time_step_kernel(cfg, device, prompt, K: int) -> dict:
    """The same decode with every step run as ONE persistent cooperative kernel (grid barriers between dependent ops) instead
    of the CUDA graph of one kernel per op, and where its time goes (CTA 0's own work per phase kind, and its waits at the grid
    barriers). The graph is the default because it measures faster; this is the record of by how much."""
    import torch

    import numpy as np

    b = build_backend(cfg, PROMPT_LEN + K + 24, 1, 0, device, step_mode="kernel")
    tok = 0
    mine, mine_first = np.zeros(cfg.vocab, np.float32), np.zeros(cfg.vocab, np.float32)
    for pos, t in enumerate(prompt):
        tok, _ = b.step(int(t), pos, mine_first if pos == 0 else mine if pos == PROMPT_LEN - 1 else None)
    out, _ = b.decode(tok, PROMPT_LEN, 8)
    b.phase_times(True)
    out, ms = b.decode(int(out[-1]), PROMPT_LEN + 8, K)
    pt = b.phase_times(False)
    res = {"tokens_per_s": K / (ms * 1e-3), "ms_per_step": ms / K, "launches_per_step": b.launches_per_step,
           "us_per_step_by_phase_kind": {k: {"work": round(w / K * 1e3, 1), "barrier_wait": round(bw / K * 1e3, 1), "phases": round(n / K, 1)}
                                         for k, (w, bw, n) in pt.items()}}
    b.close()
    torch.cuda.empty_cache()
    # How far two correct single-GPU paths part on this random-init model: the graph and this kernel differ only in the
    # order of a few float sums (split-KV merge, GEMV row tiling is the same), yet a last-bit difference flips a Q8 or f16
    # rounding here and there and 32 random layers amplify it. The scale against which the sharded runs' logits are read.
    g = build_backend(cfg, PROMPT_LEN + 8, 1, 0, device)
    want, want_first = np.zeros(cfg.vocab, np.float32), np.zeros(cfg.vocab, np.float32)
    for pos, t in enumerate(prompt):
        g.step(int(t), pos, want_first if pos == 0 else want if pos == PROMPT_LEN - 1 else None)
    g.close()
    torch.cuda.empty_cache()
    res["last_prompt_token_logits_vs_graph"] = {"max_abs_diff": float(np.abs(mine - want).max()), "logit_range": [float(want.min()), float(want.max())],
                                                "argmax_identical": bool(mine.argmax() == want.argmax())}
    # the first position already: no cache, no history, only the int8 roundings of the activations between 32 random layers
    res["first_position_logits_vs_graph"] = {"max_abs_diff": float(np.abs(mine_first - want_first).max())}
    return res


def time_f32_head(device, prompt, K: int) -> dict:
    """The Llama-3-8B shape with the output head and the embedding kept in f32 (the literal reading of the benchmark
    definition: 2.10 GB more per token through the f32 GEMV)."""
    import torch

    from amd_c_b200 import gguf

    cfg = gguf.config("llama3-8b-f32head")
    b = build_backend(cfg, PROMPT_LEN + K + 24, 1, 0, device)
    tok = 0
    for pos, t in enumerate(prompt[:16]):
        tok, _ = b.step(int(t), pos)
    out, _ = b.decode(tok, 16, 8)
    out, ms = b.decode(int(out[-1]), 24, K)
    res = {"workload": "the same model with f32 embedding and output head", "tokens_per_s": K / (ms * 1e-3), "ms_per_step": ms / K,
           "weight_gb_per_token": b.weight_bytes_per_token / 1e9, "step_weight_gb_per_s": b.weight_bytes_per_token / (ms / K * 1e-3) / 1e9}
    b.close()
    torch.cuda.empty_cache()
    return res


def time_long_context(device, positions: int = 32768, n_gen: int = 64) -> dict:
    """The 27B-class dense Q4_K_M model (64 layers, d_model 5120, 40 / 8 heads of 128, FFN 17408): `positions` seeded
    prompt ids prefilled in chunks of 256, then greedy decode with the split-KV attention reading the whole cache every
    step. Run with --long-context (about a minute); not part of the default line."""
    import numpy as np
    import torch

    from amd_c_b200 import gguf
    from amd_c_b200.backend import Backend, prefill

    cfg = gguf.config("dense-27b-q4km")
    tensors = gguf.make_model_device(cfg, seed=0)
    b = Backend(cfg, positions + n_gen + 8, T=256, device_tensors=tensors, device=device)
    del tensors
    torch.cuda.empty_cache()
    prompt = np.random.default_rng(4).integers(0, cfg.vocab, positions)
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    tok = prefill(b, prompt, 256)
    torch.cuda.synchronize(device)
    dt = time.perf_counter() - t0
    out, _ = b.decode(tok, positions, 8)
    out, ms = b.decode(int(out[-1]), positions + 8, n_gen - 8)
    n = n_gen - 8
    kv_bytes = 2.0 * (positions + n_gen // 2) * cfg.n_kv * cfg.hd * 2 * cfg.n_layer
    res = {"workload": f"27B-class dense Q4_K_M, 64 layers, {positions} positions prefilled in chunks of 256, then {n} timed greedy tokens, f16 KV cache",
           "prefill_tokens_per_s": positions / dt, "decode_tokens_per_s": n / (ms * 1e-3), "decode_ms_per_step": ms / n,
           "weight_gb_per_token": b.weight_bytes_per_token / 1e9, "kv_gb_per_token": kv_bytes / 1e9,
           "step_gb_per_s": (b.weight_bytes_per_token + kv_bytes) / (ms / n * 1e-3) / 1e9}
    b.close()
    torch.cuda.empty_cache()
    return res


def time_long_context_tp(device, group, rank: int, world: int, positions: int = 32768, n_gen: int = 40) -> dict | None:
    """The same 27B-class model sharded over the ranks of `group` (8 KV heads, FFN 17408: 2 or 4 ranks; at 8 the K-quant
    column slices of ffn_down would not be whole super-blocks): prefill in chunks of 256 (every stop of a chunk one exchange
    over 256 x 5120 floats), then greedy decode; device time of the slowest rank."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from amd_c_b200 import gguf
    from amd_c_b200.backend import Backend
    from amd_c_b200.tp import TensorParallelBackend

    cfg = gguf.config("dense-27b-q4km")
    if cfg.n_kv % world or (cfg.ffn // world) % 256:
        return None
    tensors = gguf.make_model_device(cfg, seed=0, device=device)
    b = Backend(cfg, positions + n_gen + 8, T=256, device_tensors=tensors, tp=world, rank=rank, device=device)
    del tensors
    torch.cuda.empty_cache()
    tpb = TensorParallelBackend(b, group)
    prompt = np.random.default_rng(4).integers(0, cfg.vocab, positions).astype(np.uint32)
    torch.cuda.synchronize(device)
    dist.barrier(group=group)
    t0 = time.perf_counter()
    tok = 0
    for p0 in range(0, positions, 256):
        tok = int(tpb.run(prompt[p0: p0 + 256], p0, last_only=True)[-1])
    torch.cuda.synchronize(device)
    dt = time.perf_counter() - t0
    out = tpb.decode(tok, positions, 8)
    out, ms = tpb.decode(int(out[-1]), positions + 8, n_gen - 8, timed=True)
    t = torch.tensor([ms, dt * 1e3], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    ms, dt_ms = float(t[0]), float(t[1])
    n = n_gen - 8
    kv_bytes = 2.0 * (positions + n_gen // 2) * cfg.n_kv * cfg.hd * 2 * cfg.n_layer
    res = {"workload": f"27B-class dense Q4_K_M sharded over {world} GPUs, {positions} positions prefilled in chunks of 256, then {n} timed greedy tokens",
           "prefill_tokens_per_s": positions / (dt_ms * 1e-3), "decode_tokens_per_s": n / (ms * 1e-3), "decode_ms_per_step": ms / n,
           "weight_gb_per_token_per_gpu": b.weight_bytes_per_token / 1e9, "kv_gb_per_token_per_gpu": kv_bytes / world / 1e9}
    tpb.close()
    torch.cuda.empty_cache()
    return res


def run_ours_single(args, cfg) -> dict:
    import numpy as np
    import torch

    from amd_c_b200 import _lib

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    K, W = args.steps, args.warmup
    n_ctx = PROMPT_LEN + 2 * (K + W) + 8
    b = build_backend(cfg, n_ctx, 1, 0, dev)
    lib = _lib.load()
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg.vocab, PROMPT_LEN)
    tok = 0
    for pos, t in enumerate(prompt):  # the prompt, token by token (the reference has no Q4_0 prompt kernel either)
        tok, _ = b.step(int(t), pos)
    pos = PROMPT_LEN
    # ---- device-resident decode: W warm-up steps, then K timed steps
    out, _ = b.decode(tok, pos, W)
    tok, pos = int(out[-1]), pos + W
    torch.cuda.synchronize()
    with ClockSampler(0) as cs:
        l0 = lib.ie_b200_launch_count()
        out, ms = b.decode(tok, pos, K)
        launches = lib.ie_b200_launch_count() - l0
        tok, pos = int(out[-1]), pos + K
        # ---- end to end: token in from the host, argmax out to the host, every step
        for _ in range(W):
            tok, _ = b.step(tok, pos)
            pos += 1
        t0 = time.perf_counter()
        for _ in range(K):
            tok, _ = b.step(tok, pos)
            pos += 1
        e2e_s = time.perf_counter() - t0
    clocks = cs.summary()
    gem = time_gemvs(b)
    peak, peak_src = measured_peaks()
    achieved = gem["bytes"] / (gem["ms_per_pass"] * 1e-3) / 1e9
    res = {
        "value": K / (ms * 1e-3), "ms_per_step": ms / K, "gpu_launches": int(launches),
        "e2e": {"value": K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 12},
        "roofline": {"bound": "hbm", "kernel": "gemv (Q4_0 x Q8, decode)", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": f"{peak_src} copy bandwidth", "frac_of_nominal_8000": achieved / 8000.0,
                     "traffic": gem["bytes"] * NCU_TRAFFIC_RATIO / max(1, gem["launches"]),
                     "traffic_note": "dram bytes per launch: the ncu capture of one 14336x4096 launch (1.002 x its algorithmic bytes) scaled to the average launch",
                     "achieved_best_of_repeats": gem["bytes"] / (gem["ms_per_pass_min"] * 1e-3) / 1e9, "repeats": gem["repeats"],
                     "algorithmic_bytes_per_launch": gem["bytes"] / max(1, gem["launches"]),
                     "launches_per_step": gem["launches"], "avg_launch_us": gem["ms_per_pass"] * 1e3 / max(1, gem["launches"]),
                     "algorithmic_bytes_per_step": gem["bytes"],
                     "scope": "all GEMV launches of one decode step, back to back in step order (dependent chain, real matrices)"},
        "step_weight_gb_per_s": b.weight_bytes_per_token / (ms / K * 1e-3) / 1e9,
        "launches_per_step": b.launches_per_step, "clocks": clocks,
    }
    b.close()
    torch.cuda.empty_cache()
    res["step_mode"] = "graph (one kernel per op, programmatic dependent launch)"
    res["step_kernel"] = time_step_kernel(cfg, dev, prompt, min(K, 128))
    res["roofline"]["gemv_sweep"] = time_gemv_sweep(dev, peak)
    res["attention"] = time_attention(dev, peak)
    res["prefill_gemm"] = time_prefill_gemm(dev)
    if not args.quick:
        res["llama3_8b_f32_head"] = time_f32_head(dev, prompt, min(K, 64))
        res["qwen2_7b_q4km"] = time_qwen2_prefill(dev)
        res["dense_27b_q4km_32k"] = time_long_context(dev)
    return res


def run_ours_tp(args, cfg, rank: int, world: int) -> dict | None:
    """Tensor-parallel decode under torchrun: one process per GPU, NCCL for the rendezvous, the per-half-layer
    sums through the peer-memory all-reduce kernel (amd_c_b200/tp.py). Returns the result dict on rank 0."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from amd_c_b200 import _lib
    from amd_c_b200.tp import TensorParallelBackend

    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    K, W = args.steps, max(args.warmup, 32)  # at least 32 warm-up tokens: they are also the tokens compared with one GPU
    n_ctx = PROMPT_LEN + 2 * (K + W) + 8
    b = build_backend(cfg, n_ctx, world, rank, dev)
    tpb = TensorParallelBackend(b, dist.group.WORLD)
    lib = _lib.load()
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg.vocab, PROMPT_LEN)
    tok = 0
    my_logits, my_first = np.zeros(b.vocab_l, np.float32), np.zeros(b.vocab_l, np.float32)
    for pos, t in enumerate(prompt):
        tok = tpb.step(int(t), pos, my_first if pos == 0 else my_logits if pos == PROMPT_LEN - 1 else None)
    pos = PROMPT_LEN
    first_tok = tok
    out = tpb.decode(tok, pos, W)
    tok, pos = int(out[-1]), pos + W
    torch.cuda.synchronize()
    def gathered(mine):  # rank r holds logits [r * vocab / world, (r + 1) * vocab / world)
        sl = torch.from_numpy(mine).to(dev)
        slices = [torch.empty_like(sl) for _ in range(world)]
        dist.all_gather(slices, sl)
        return torch.cat(slices).cpu().numpy()

    tp_logits, tp_first = gathered(my_logits), gathered(my_first)
    # correctness beside the timing, outside the timed region, against an unsharded engine on rank 0's GPU (the other ranks
    # wait). The sharded sums add per-rank partial rows in rank order, the unsharded engine sums a whole row at once, and the
    # f16 KV cache turns a last-bit difference into a different cache entry here and there: the logits agree to about 1e-2,
    # so a choice between two tokens whose logits lie closer than that may differ. Reported, not asserted: the logits of
    # the last prompt token, the free-running common prefix, and the next-token choices with the unsharded engine fed the
    # sharded run's tokens (each disagreement with the margin by which the unsharded logits prefer their own choice).
    identical = None
    if rank == 0:
        single = build_backend(cfg, n_ctx, 1, 0, dev)
        want, want_first = np.zeros(cfg.vocab, np.float32), np.zeros(cfg.vocab, np.float32)
        t1 = 0
        for p1, t in enumerate(prompt):
            t1, _ = single.step(int(t), p1, want_first if p1 == 0 else want if p1 == PROMPT_LEN - 1 else None)
        mine_seq = [first_tok] + [int(x) for x in out]
        srt = np.sort(want)
        first = {"max_abs_diff": float(np.abs(tp_logits - want).max()), "logit_range": [float(srt[0]), float(srt[-1])],
                 "top1_minus_top2": float(srt[-1] - srt[-2]), "argmax_identical": bool(t1 == first_tok)}
        agree, margins, nxt = int(t1 == first_tok), [], np.zeros(cfg.vocab, np.float32)
        if t1 != first_tok:
            margins.append(float(want[t1] - want[first_tok]))
        for i in range(W):  # teacher-forced: the same history on both sides
            c1, _ = single.step(mine_seq[i], PROMPT_LEN + i, nxt)
            if c1 == mine_seq[i + 1]:
                agree += 1
            else:
                margins.append(float(nxt[c1] - nxt[mine_seq[i + 1]]))
        single.close()
        single = build_backend(cfg, n_ctx, 1, 0, dev)
        for p1, t in enumerate(prompt):
            t1, _ = single.step(int(t), p1)
        o1, _ = single.decode(t1, PROMPT_LEN, W)
        single.close()
        torch.cuda.empty_cache()
        want_seq = [t1] + [int(x) for x in o1]
        prefix = next((i for i, (a, b) in enumerate(zip(mine_seq, want_seq)) if a != b), len(want_seq))
        identical = {"first_position_logits_max_abs_diff": float(np.abs(tp_first - want_first).max()),  # before any rounding can have flipped: the float order of the sharded sums alone
                     "tokens_compared": len(want_seq), "identical_prefix": prefix, "same_history_choices_identical": agree,
                     "margins_at_disagreements": margins, "last_prompt_token_logits": first}
    dist.barrier()
    with ClockSampler(local) as cs:
        torch.cuda.synchronize()
        l0 = lib.ie_b200_launch_count()
        out, ms = tpb.decode(tok, pos, K, timed=True)
        launches = lib.ie_b200_launch_count() - l0
        tok, pos = int(out[-1]), pos + K
        for _ in range(W):
            tok = tpb.step(tok, pos)
            pos += 1
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(K):
            tok = tpb.step(tok, pos)
            pos += 1
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    clocks = cs.summary()
    t = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)  # the slowest rank's device time is the job's time
    ms, e2e_ms = float(t[0]), float(t[1])
    gem = time_gemvs(b)
    # the same chain with the exchanges: every K-split GEMV pushes its rows and the one-CTA kernel behind it reduces, adds the
    # residual, normalises and quantises (all ranks replay in step; the difference per stop is what an exchange costs, waiting
    # for the slowest rank included)
    from amd_c_b200.backend import OP_ALLREDUCE, OP_GEMV, OP_RMSNORM
    dist.barrier()
    with_stops = time_gemvs(b, mask=(1 << OP_GEMV) | (1 << OP_ALLREDUCE) | (1 << OP_RMSNORM))
    n_stops = sum(1 for o in b.ops if o.kind == OP_ALLREDUCE)
    g = torch.tensor([gem["ms_per_pass"], with_stops["ms_per_pass"]], dtype=torch.float64, device=dev)
    dist.all_reduce(g, op=dist.ReduceOp.MAX)
    peak, peak_src = measured_peaks()
    achieved = gem["bytes"] / (float(g[0]) * 1e-3) / 1e9  # per GPU: this rank's shard bytes over the slowest rank's time
    res = None
    if rank == 0:
        res = {
            "value": K / (ms * 1e-3), "ms_per_step": ms / K, "gpu_launches": int(launches),
            "e2e": {"value": K / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 12 * world, "d2h_bytes_per_step": 8 * world},
            "roofline": {"bound": "hbm", "kernel": "gemv (Q4_0 x Q8, decode), per GPU", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": f"{peak_src} copy bandwidth", "frac_of_nominal_8000": achieved / 8000.0,
                         "traffic": None, "launches_per_step": gem["launches"], "algorithmic_bytes_per_step": gem["bytes"]},
            "allreduce": {**tpb.describe(), "us_per_stop": (float(g[1]) - float(g[0])) * 1e3 / max(1, n_stops),
                          "us_per_stop_note": "GEMVs + exchanges + norms of a step as a dependent chain, minus the GEMVs alone, per exchange"},
            "clocks": clocks, "tp_tokens_identical_prefix": identical,
        }
    tpb.close()
    torch.cuda.empty_cache()
    dist.barrier()
    if not args.quick:  # the long-context model sharded the same way (2 or 4 ranks), every rank takes part
        long_tp = time_long_context_tp(dev, dist.group.WORLD, rank, world)
        if res is not None and long_tp is not None:
            res["dense_27b_q4km_32k"] = long_tp
    dist.barrier()
    dist.destroy_process_group()
    return res


# ------------------------------------------------------------------ profiler cases
# Small stand-alone cases of the hot kernels, sized for a profiler: few launches, a few GB on the device at most,
# inputs larger than L2 where DRAM figures matter. Each prints the CUDA-event time per launch; under ncu select the
# kernel with -k regex:<name>.
#   python bench.py --case gemv [rows cols [q4_0|q4_k|q6_k [launches]]]   decode GEMV on rotating copies of one matrix
#   python bench.py --case gemm [rows cols T [q4_0|q4_k|q6_k]]             prompt-chunk GEMM, int8 mma.sync kernel
#   python bench.py --case gemm_tc [rows cols T [q4_0|q4_k|q6_k]]          prompt-chunk GEMM, tcgen05 kernel
#   python bench.py --case attn [positions [launches]]                     decode attention, Llama-3-8B heads, f16 cache
#   python bench.py --case step [config [position [steps]]]               whole decode steps as plain launches (no graph)

def run_case(argv) -> None:
    import numpy as np  # noqa: F401
    import torch

    from amd_c_b200 import gguf, synth
    from amd_c_b200 import kernels as K
    from amd_c_b200.backend import Backend

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


    def case_gemm_tc(rows=37888, cols=3584, T=256, kind="q4_k"):
        dev = torch.device("cuda:0")
        gen = torch.Generator(device=dev).manual_seed(0)
        m = _matrix(KINDS[kind], int(rows), int(cols), gen, dev)
        xq = K.quant_q8(torch.randn(int(T), int(cols), device=dev, generator=gen))
        us = _timed(lambda i: K.gemm_tc(m, xq), 5)
        print(f"gemm_tc {kind} {rows}x{cols} T={T}: {us:.1f} us per call (expansion of the activations + GEMM), {2.0 * int(rows) * int(cols) * int(T) / us / 1e6:.1f} TFLOP/s")

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


    cases = {"gemv": case_gemv, "gemm": case_gemm, "gemm_tc": case_gemm_tc, "attn": case_attn, "step": case_step}
    if not argv or argv[0] not in cases:
        sys.exit("bench.py --case gemv|gemm|gemm_tc|attn|step [arguments]")
    cases[argv[0]](*argv[1:])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llama3-8b")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--long-context", action="store_true", help="(kept for old command lines: the 27B-class model at 32768 positions is part of the default run)")
    ap.add_argument("--quick", action="store_true", help="skip the other configurations (f32 head, Qwen2-7B prompt, 27B-class long context)")
    ap.add_argument("--case", nargs="+", default=None, help="run one small profiler case instead of the benchmark: gemv|gemm|attn|step [arguments]")
    args = ap.parse_args()
    if args.case:
        run_case(args.case)
        return
    if args.warmup < 3:
        args.warmup = 3

    from amd_c_b200 import gguf

    cfg = gguf.config(args.config)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank)
        return
    if world != args.gpus and world > 1:
        args.gpus = world
    if args.gpus > 1 and world == 1:
        sys.exit("bench.py --gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    # Exactly one JSON line goes to stdout: while the benchmark runs, file descriptor 1 points at stderr, so that
    # banners that libraries write straight to it (NCCL's version line) do not land in front of the result.
    sys.stdout.flush()
    out_fd = os.dup(1)
    os.dup2(2, 1)
    try:
        res = run_ours_single(args, cfg) if world == 1 else run_ours_tp(args, cfg, rank, world)
    finally:
        sys.stdout.flush()
        os.dup2(out_fd, 1)
        os.close(out_fd)
    if rank != 0:
        return
    line = {"metric": METRIC, "value": res.pop("value"), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": res.pop("ms_per_step"), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 dot4 + f32 accumulate", "data": "synthetic", "config": workload_config(cfg, world)}
    line.update(res)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
