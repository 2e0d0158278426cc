"""Seeded synthetic weights in GGUF block formats.

Q4_0 follows the benchmark definition: weights drawn N(0, sigma) from a fixed
seed; per block of 32, d = f16(amax / 7) and the 4-bit code is
round(w / d) + 8 clamped to 0..15 (weight j in the low nibble of byte j,
weight j + 16 in the high nibble, 18 bytes per block: f16 d, 16 bytes).
Q4_K / Q6_K super-blocks are random codes and sub-scales with small fixed f16
super-scales, so values are bounded and exactly representable.

numpy versions serve the tests; the torch versions build large matrices on
the GPU (same definition, torch's generator).
"""
from __future__ import annotations

import numpy as np

GGML_F32, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 0, 2, 8, 12, 14
BLOCK_BYTES = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}


def gguf_nbytes(ggml_type: int, rows: int, cols: int) -> int:
    if ggml_type == GGML_F32:
        return rows * cols * 4
    n, b = BLOCK_BYTES[ggml_type]
    return rows * cols // n * b


def q4_0_from_weights(w: np.ndarray) -> np.ndarray:
    """f32 [rows, cols] -> GGUF Q4_0 bytes uint8 [rows, cols/32, 18]."""
    rows, cols = w.shape
    nb = cols // 32
    wb = w.reshape(rows, nb, 32).astype(np.float32)
    amax = np.abs(wb).max(axis=2)
    d = (amax / np.float32(7.0)).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(df[..., None] != 0, np.round(wb / df[..., None]), 0.0)
    q = np.clip(q + 8, 0, 15).astype(np.uint8)
    blk = np.empty((rows, nb, 18), dtype=np.uint8)
    blk[:, :, 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    blk[:, :, 2:] = q[:, :, :16] | (q[:, :, 16:] << 4)
    return blk


def q4_0_normal(rng: np.random.Generator, rows: int, cols: int, sigma: float = 0.02) -> np.ndarray:
    return q4_0_from_weights(rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(sigma))


def q8_0_normal(rng: np.random.Generator, rows: int, cols: int, sigma: float = 0.02) -> np.ndarray:
    """GGUF Q8_0 bytes uint8 [rows, cols/32, 34] of N(0, sigma) weights: per block d = f16(amax / 127), q = round(w / d)."""
    nb = cols // 32
    wb = (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(sigma)).reshape(rows, nb, 32)
    d = (np.abs(wb).max(axis=2) / np.float32(127.0)).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(df[..., None] != 0, np.round(wb / df[..., None]), 0.0)
    blk = np.empty((rows, nb, 34), dtype=np.uint8)
    blk[:, :, 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    blk[:, :, 2:] = np.clip(q, -127, 127).astype(np.int8).view(np.uint8)
    return blk


def q4_k_random(rng: np.random.Generator, rows: int, cols: int, scale: float = 0.02) -> np.ndarray:
    """GGUF Q4_K bytes uint8 [rows, cols/256, 144]: random scales/codes, fixed small f16 d and dmin."""
    nsb = rows * cols // 256
    b = rng.integers(0, 256, size=(nsb, 144), dtype=np.uint8)
    b[:, 0:2] = np.full(nsb, scale / 16.0 / 63.0 * 4, np.float16).view(np.uint8).reshape(nsb, 2)
    b[:, 2:4] = np.full(nsb, scale / 63.0 * 2, np.float16).view(np.uint8).reshape(nsb, 2)
    return b.reshape(rows, cols // 256, 144)


def q6_k_random(rng: np.random.Generator, rows: int, cols: int, scale: float = 0.02) -> np.ndarray:
    """GGUF Q6_K bytes uint8 [rows, cols/256, 210]: random codes, int8 sub-scales in [-40, 40), fixed small f16 d."""
    nsb = rows * cols // 256
    b = rng.integers(0, 256, size=(nsb, 210), dtype=np.uint8)
    b[:, 192:208] = rng.integers(-40, 40, size=(nsb, 16)).astype(np.int8).view(np.uint8)
    b[:, 208:210] = np.full(nsb, scale / 32.0 / 40.0 * 4, np.float16).view(np.uint8).reshape(nsb, 2)
    return b.reshape(rows, cols // 256, 210)


def make_gguf_bytes(ggml_type: int, rng: np.random.Generator, rows: int, cols: int, sigma: float = 0.02) -> np.ndarray:
    if ggml_type == GGML_Q4_0:
        return q4_0_normal(rng, rows, cols, sigma)
    if ggml_type == GGML_Q8_0:
        return q8_0_normal(rng, rows, cols, sigma)
    if ggml_type == GGML_Q4_K:
        return q4_k_random(rng, rows, cols, sigma)
    if ggml_type == GGML_Q6_K:
        return q6_k_random(rng, rows, cols, sigma)
    if ggml_type == GGML_F32:
        return (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(sigma)).view(np.uint8)
    raise ValueError(ggml_type)


# ---- torch (device-side) generators for large matrices ----

def q4_0_normal_torch(gen, rows: int, cols: int, sigma: float = 0.02, device="cuda", chunk_rows: int = 8192):
    """GGUF Q4_0 bytes as a uint8 CUDA tensor [rows, cols/32, 18], built in row chunks on the device."""
    import torch

    nb = cols // 32
    out = torch.empty((rows, nb, 18), dtype=torch.uint8, device=device)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        w = torch.randn((r1 - r0, nb, 32), generator=gen, device=device, dtype=torch.float32) * sigma
        d = (w.abs().amax(dim=2) / 7.0).to(torch.float16)
        df = d.to(torch.float32).unsqueeze(-1)
        q = torch.where(df != 0, torch.round(w / df), torch.zeros_like(w))
        q = (q + 8).clamp_(0, 15).to(torch.uint8)
        out[r0:r1, :, 0:2] = d.view(torch.uint8).reshape(r1 - r0, nb, 2)
        out[r0:r1, :, 2:] = q[:, :, :16] | (q[:, :, 16:] << 4)
    return out


def q8_0_normal_torch(gen, rows: int, cols: int, sigma: float = 0.02, device="cuda", chunk_rows: int = 8192):
    """GGUF Q8_0 bytes as a uint8 CUDA tensor [rows, cols/32, 34] of N(0, sigma) weights, built in row chunks on the device."""
    import torch

    nb = cols // 32
    out = torch.empty((rows, nb, 34), dtype=torch.uint8, device=device)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        w = torch.randn((r1 - r0, nb, 32), generator=gen, device=device, dtype=torch.float32) * sigma
        d = (w.abs().amax(dim=2) / 127.0).to(torch.float16)
        df = d.to(torch.float32).unsqueeze(2)
        q = torch.where(df != 0, torch.round(w / df), torch.zeros_like(w)).clamp_(-127, 127).to(torch.int8)
        out[r0:r1, :, 0:2] = d.view(torch.uint8).reshape(r1 - r0, nb, 2)
        out[r0:r1, :, 2:] = q.view(torch.uint8)
    return out


def k_random_torch(ggml_type: int, gen, rows: int, cols: int, scale: float = 0.02, device="cuda"):
    """GGUF Q4_K / Q6_K bytes as a uint8 CUDA tensor (same construction as the numpy versions)."""
    import torch

    nsb = rows * cols // 256
    if ggml_type == GGML_Q4_K:
        b = torch.randint(0, 256, (nsb, 144), generator=gen, device=device, dtype=torch.uint8)
        hdr = np.concatenate([np.full(1, scale / 16.0 / 63.0 * 4, np.float16).view(np.uint8), np.full(1, scale / 63.0 * 2, np.float16).view(np.uint8)])
        b[:, 0:4] = torch.from_numpy(hdr).to(device)
        return b.reshape(rows, cols // 256, 144)
    b = torch.randint(0, 256, (nsb, 210), generator=gen, device=device, dtype=torch.uint8)
    sc = torch.randint(-40, 40, (nsb, 16), generator=gen, device=device, dtype=torch.int8)
    b[:, 192:208] = sc.view(torch.uint8)
    b[:, 208:210] = torch.from_numpy(np.full(1, scale / 32.0 / 40.0 * 4, np.float16).view(np.uint8)).to(device)
    return b.reshape(rows, cols // 256, 210)
