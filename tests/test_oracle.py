"""The oracle (C restatement) against the reference: golden fixtures made by
the reference's own src/cpu.c, the known-answer construction of its
tests/kernel_test.c, and (where it is built) the compiled reference itself."""
import hashlib
import tempfile
from pathlib import Path

import numpy as np
import pytest

from amd_c_b200 import gguf, synth
from conftest import GOLDEN, bits
from oracle.oracle import MAT_Q4, OracleModel

sys_path_note = None
Q4_SHAPES = [(1, 1), (7, 3), (9, 11), (8, 32), (13, 33), (17, 36), (5, 64), (3, 100), (2, 511)]
K_SHAPES = [(3, 8), (9, 16), (8, 40), (5, 112), (2, 448)]
KINDS = [(synth.GGML_Q4_0, Q4_SHAPES, "q4_0"), (synth.GGML_Q4_K, K_SHAPES, "q4_k"), (synth.GGML_Q6_K, K_SHAPES, "q6_k"),
         (synth.GGML_Q8_0, Q4_SHAPES, "q8_0")]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_quant_q8_golden(ora, golden_kernels):
    g = golden_kernels
    q = ora.quant_q8(g["quant_x"])
    assert (q == g["quant_q"]).all()
    nb = g["quant_x"].size // 32
    # the zero block has d = 0, q = 0, asum = 0
    assert q[32:64].max() == 0 and q[32 * nb + 4: 32 * nb + 8].view(np.float32)[0] == 0.0


@pytest.mark.parametrize("typ,shapes,tag", KINDS)
def test_repack_and_gemv_golden(ora, golden_kernels, typ, shapes, tag):
    g = golden_kernels
    for rows, nb in shapes:
        cols, key = nb * 32, f"{tag}_{rows}x{nb}"
        kind, qw, qs = ora.repack(typ, g[key + "_raw"], rows, cols)
        assert (sha(qw) + sha(qs)).encode() == g[key + "_sha"].tobytes(), key  # the reference's repacked arrays, byte for byte
        y = ora.gemv(kind, qw, qs, rows, cols, ora.quant_q8(g[key + "_x"]))
        assert (bits(y) == bits(g[key + "_y"])).all(), key


def test_q4_gemv_known_answer(ora):
    """As the reference's kernel test: the GEMV against a double-precision
    element-wise dot taken from the GGUF bytes; nibbles survive the repack;
    the stored block sum is the sum of the 32 int8."""
    rng = np.random.default_rng(7)
    worst = 0.0
    for rows, nb in Q4_SHAPES:
        cols = nb * 32
        raw = np.zeros((rows, nb, 18), np.uint8)
        raw[:, :, 0:2] = (0.01 + 0.02 * rng.integers(0, 100, (rows, nb)) / 100.0).astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
        raw[:, :, 2:] = rng.integers(0, 256, (rows, nb, 16), dtype=np.uint8)
        kind, qw, qs = ora.repack(synth.GGML_Q4_0, raw, rows, cols)
        assert kind == MAT_Q4
        nib = np.concatenate([raw[:, :, 2:] & 15, raw[:, :, 2:] >> 4], axis=2).astype(np.int64)  # weight j of every block
        words = qw.reshape(rows, nb, 4)
        for j in range(32):
            got = (words[:, :, (j & 15) >> 2] >> (8 * (j & 3) + 4 * (j >> 4))) & 15
            assert (got == nib[:, :, j]).all()
        x = (rng.uniform(-1, 1, cols) * np.where(np.arange(cols) % 7 == 0, 3.0, 1.0)).astype(np.float32)
        xq = ora.quant_q8(x)
        qa = xq[: 32 * nb].view(np.int8).astype(np.int64).reshape(nb, 32)
        da = xq[32 * nb: 36 * nb].view(np.float32).astype(np.float64)
        asum = xq[36 * nb:].view(np.uint32)
        assert (asum == (qa.sum(axis=1) & 0xFFFFFFFF).astype(np.uint32)).all()
        y = ora.gemv(kind, qw, qs, rows, cols, xq)
        d = raw[:, :, 0:2].copy().view(np.float16).astype(np.float64).reshape(rows, nb)
        terms = d * da[None, :] * ((nib - 8) * qa[None, :, :]).sum(axis=2)
        ref, mag = terms.sum(axis=1), np.abs(terms).sum(axis=1)
        err = np.abs(ref - y) / np.where(mag > 0, mag, 1.0)
        worst = max(worst, err.max())
        dots = ora.block_dots_q4(qw, rows, nb, xq).reshape(rows, nb)
        assert (dots == ((nib - 8) * qa[None]).sum(axis=2)).all()
    assert worst < 1e-5  # the reference's own tolerance


@pytest.mark.parametrize("name,fname,n_ctx", [("tiny", "tiny.npz", 512), ("tiny-k", "tiny_k.npz", 256), ("tiny-q8", "tiny_q8.npz", 256)])
def test_model_golden(ora, name, fname, n_ctx):
    """Greedy ids, logits and per-layer outputs of the synthetic tiny models: bit-exact with the reference CPU backend."""
    g = np.load(GOLDEN / fname)
    cfg = gguf.make_model(gguf.config(name), seed=int(g["seed"]))
    with tempfile.TemporaryDirectory() as td:
        p = Path(td) / "m.gguf"
        gguf.write_gguf(p, cfg)
        assert hashlib.sha256(p.read_bytes()).hexdigest().encode() == g["gguf_sha"].tobytes(), "the seeded generator changed"
        back = gguf.read_gguf(p)
        assert all((back.tensors[k].raw() == cfg.tensors[k].raw()).all() for k in cfg.tensors)
    m = OracleModel(ora, cfg, n_ctx)
    m.enable_trace()
    ids = list(g["ids"])
    tok = ids[0]
    for pos in range(len(ids) - 1):
        nxt, lg = m.step(int(tok), pos)
        if pos < len(g["logits"]):
            assert (bits(lg) == bits(g["logits"][pos])).all(), pos
        if g["traces"].ndim == 3 and pos < len(g["traces"]):
            assert (bits(m.trace) == bits(g["traces"][pos])).all(), pos
        if pos + 1 >= 3:
            assert nxt == ids[pos + 1], pos
        tok = ids[pos + 1]
    m.close()


def test_oracle_equals_compiled_reference(ora, ref):
    """Fresh seeded inputs through both: quantiser, repacks, GEMVs (skipped where the reference was never built)."""
    rng = np.random.default_rng(99)
    x = rng.standard_normal(4096).astype(np.float32)
    assert (ora.quant_q8(x) == ref.quant_q8(x)).all()
    for typ, (rows, cols) in [(2, (13, 33 * 32)), (2, (2, 511 * 32)), (12, (9, 512)), (14, (9, 768)), (12, (16, 3584)), (14, (17, 2048)),
                              (8, (13, 33 * 32)), (8, (5, 2048))]:
        raw = synth.make_gguf_bytes(typ, rng, rows, cols)
        kind, qw, qs = ora.repack(typ, raw, rows, cols)
        rm = ref.mat(typ, raw, rows, cols)
        rqw, rqs = rm.arrays()
        assert rm.kind == kind and (rqw == qw).all() and (rqs == qs).all()
        xq = ora.quant_q8(rng.standard_normal(cols).astype(np.float32))
        assert (bits(ora.gemv(kind, qw, qs, rows, cols, xq)) == bits(rm.gemv(xq))).all()
        rm.free()


def test_f16_conversions(ora):
    h = np.arange(0, 65536, dtype=np.uint16)
    f = h.view(np.float16).astype(np.float32)
    ok = ~np.isnan(f)
    got = np.array([ora.lib.ora_f16_to_f32(int(v)) for v in h[::37]], np.float32)
    assert (bits(got)[ok[::37]] == bits(f[::37])[ok[::37]]).all()
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(2000).astype(np.float32) * 10.0 ** rng.integers(-8, 5, 2000), np.float32([0, 65504, 65520, 1e-8, 6e-5])])
    want = x.astype(np.float16).view(np.uint16)
    got16 = np.array([ora.lib.ora_f32_to_f16(float(v)) for v in x], np.uint16)
    assert (got16 == want).all()
