"""Parity of the CUDA kernels (through the C ABI) with the oracle on the same
seeded inputs. Integer / byte work and the GEMV floats: bit-exact. Ops whose
reduction order differs from the CPU's (RMSNorm sum, attention): relative
tolerance 1e-4 of the output scale, written at each assertion."""
import numpy as np
import pytest

from amd_c_b200 import synth
from conftest import bits
from oracle.oracle import MAT_F32, MAT_Q4, MAT_Q4K, MAT_Q6K, MAT_Q8

pytestmark = pytest.mark.gpu

Q4_SHAPES = [(1, 1), (7, 3), (9, 11), (8, 32), (13, 33), (17, 36), (5, 64), (3, 100), (2, 511)]
K_SHAPES = [(3, 8), (9, 16), (8, 40), (5, 112), (2, 448)]
KINDS = [(synth.GGML_Q4_0, Q4_SHAPES, "q4_0"), (synth.GGML_Q4_K, K_SHAPES, "q4_k"), (synth.GGML_Q6_K, K_SHAPES, "q6_k"),
         (synth.GGML_Q8_0, Q4_SHAPES, "q8_0")]


def dev(a, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def expected_layout(kind, qw, qs, rows, cols, row_bytes):
    """The streaming layout built in numpy from the reference-form arrays."""
    nb = cols // 32
    out = np.zeros((rows, row_bytes), np.uint8)
    if kind == MAT_Q8:
        out[:, : 32 * nb] = qw.view(np.uint8).reshape(rows, 32 * nb)
        out[:, 32 * nb: 34 * nb] = qs.view(np.uint8).reshape(rows, 2 * nb)
        return out
    out[:, : 16 * nb] = qw[: rows * nb * 4].view(np.uint8).reshape(rows, 16 * nb)
    if kind == MAT_Q4:
        out[:, 16 * nb: 18 * nb] = qs.view(np.uint8).reshape(rows, 2 * nb)
    elif kind == MAT_Q4K:
        sm = qs[: rows * nb].reshape(rows, nb // 8, 8).astype(np.uint64)
        f = (sm & 63) | (((sm >> 8) & 63) << 6)
        lo = np.zeros((rows, nb // 8), np.uint64)
        for j in range(5):
            lo |= f[:, :, j] << np.uint64(12 * j)
        lo |= (f[:, :, 5] & 15) << np.uint64(60)
        w2 = (f[:, :, 5] >> 4) | (f[:, :, 6] << 8) | (f[:, :, 7] << 20)
        dd = qs[rows * nb:].reshape(rows, nb // 8, 2).astype(np.uint32)
        hdr = np.zeros((rows, nb // 8, 4), np.uint32)
        hdr[:, :, 0] = dd[:, :, 0] | (dd[:, :, 1] << 16)
        hdr[:, :, 1] = (lo & 0xFFFFFFFF).astype(np.uint32)
        hdr[:, :, 2] = (lo >> 32).astype(np.uint32)
        hdr[:, :, 3] = w2.astype(np.uint32)
        out[:, 16 * nb: 16 * nb + 2 * nb] = hdr.view(np.uint8).reshape(rows, 2 * nb)
    else:
        out[:, 16 * nb: 24 * nb] = qw[rows * nb * 4:].view(np.uint8).reshape(rows, 8 * nb)
        out[:, 24 * nb: 26 * nb] = qs[: rows * nb].view(np.uint8).reshape(rows, 2 * nb)
        out[:, 26 * nb: 26 * nb + nb // 4] = qs[rows * nb:].view(np.uint8).reshape(rows, nb // 4)
    return out


def test_quant_q8_bit_exact(ora, cuda, golden_kernels):
    from amd_c_b200 import kernels as K

    g = golden_kernels
    got = K.quant_q8(dev(g["quant_x"], cuda)).cpu().numpy().reshape(-1)
    assert (got == g["quant_q"]).all()  # the reference's own output
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((7, 14336)) * rng.choice([1e-3, 1.0, 300.0], size=(7, 1))).astype(np.float32)
    x[3, 640:672] = 0.0
    got = K.quant_q8(dev(x, cuda)).cpu().numpy()
    for t in range(x.shape[0]):
        assert (got[t] == ora.quant_q8(x[t])).all(), t


def test_quant_q8_rounding_boundaries(ora, cuda):
    """Values within a few ulps of every k + 0.5 boundary, for several scales: the kernel's reciprocal fast path
    must fall back to the exact division there and agree with the CPU quantiser bit for bit."""
    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(9)
    rows = []
    for scale in (1.0, 0.3, 0.0123, 7.77, 1e-3, 3e5, 1e-36):
        d = np.float32(np.float32(127.0 * scale) / np.float32(127.0))
        for _ in range(40):
            k = rng.integers(-126, 126, 31).astype(np.float32) + np.float32(0.5)
            v = (k * d).astype(np.float32)
            steps = rng.integers(-3, 4, 31)
            for _ in range(3):
                v = np.where(steps > 0, np.nextafter(v, np.float32(np.inf)), np.where(steps < 0, np.nextafter(v, np.float32(-np.inf)), v)).astype(np.float32)
                steps = steps - np.sign(steps)
            rows.append(np.concatenate([[np.float32(127.0 * scale)], v]).astype(np.float32))
    x = np.stack(rows)
    got = K.quant_q8(dev(x, cuda)).cpu().numpy()
    for t in range(x.shape[0]):
        assert (got[t] == ora.quant_q8(x[t])).all(), t


def test_quant_q8_empty(cuda, lib):
    assert lib.ie_b200_quant_q8(256, 256, 0, 1, 0, 0, None) == 0  # zero blocks: nothing launched, nothing read


@pytest.mark.parametrize("typ,shapes,tag", KINDS)
def test_repack_layout_and_gemv_bit_exact(ora, cuda, golden_kernels, lib, typ, shapes, tag):
    """Both repack entry points give the documented layout; block dots and GEMV match the golden outputs bit for bit."""
    from amd_c_b200 import kernels as K

    g = golden_kernels
    for rows, nb in shapes:
        cols, key = nb * 32, f"{tag}_{rows}x{nb}"
        raw = g[key + "_raw"]
        kind, qw, qs = ora.repack(typ, raw, rows, cols)
        m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
        rowb = lib.ie_b200_row_bytes(kind, cols)
        want = expected_layout(kind, qw, qs, rows, cols, rowb)
        got = m.data.cpu().numpy()[: rows * rowb].reshape(rows, rowb)
        used = {MAT_Q4: 18 * nb, MAT_Q8: 34 * nb, MAT_Q4K: 18 * nb, MAT_Q6K: 26 * nb + nb // 4}[kind]
        assert (got[:, :used] == want[:, :used]).all(), key
        m2 = K.Mat.from_ref(kind, dev(qw, cuda), dev(qs, cuda), rows, cols)
        assert (m2.data.cpu().numpy()[: rows * rowb].reshape(rows, rowb)[:, :used] == want[:, :used]).all(), key
        xq = ora.quant_q8(g[key + "_x"])
        y = K.gemv(m, dev(xq, cuda).reshape(1, -1)).cpu().numpy().reshape(-1)
        assert (bits(y) == bits(g[key + "_y"])).all(), key
        if kind == MAT_Q4:
            d = K.block_dots(m, dev(xq, cuda)).cpu().numpy()
            assert (d == ora.block_dots_q4(qw, rows, nb, xq)).all(), key
        if kind == MAT_Q8:
            d = K.block_dots(m, dev(xq, cuda)).cpu().numpy()
            assert (d == ora.block_dots_q8(qw, rows, nb, xq)).all(), key


@pytest.mark.parametrize("typ,rows,cols,ranges,c0,c1", [
    (synth.GGML_Q4_0, 96, 1024, [(8, 16), (40, 8), (72, 24)], 0, 1024),    # q / k / v heads of a merged matrix
    (synth.GGML_Q4_0, 64, 1024, [(0, 64)], 352, 352 + 160),                # a column slice that is not a multiple of 8 blocks
    (synth.GGML_Q4_K, 48, 1536, [(0, 48)], 512, 1280),
    (synth.GGML_Q6_K, 40, 2048, [(0, 40)], 1024, 2048),
    (synth.GGML_Q6_K, 40, 1024, [(4, 9), (20, 20)], 256, 768),             # rows and columns at once
    (synth.GGML_F32, 512, 512, [(256, 256)], 0, 512),                      # a vocabulary slice of an f32 head
    (synth.GGML_Q8_0, 64, 1024, [(3, 20), (40, 24)], 96, 96 + 480),
])
def test_mat_part_is_the_repack_of_the_slice(cuda, lib, typ, rows, cols, ranges, c0, c1):
    """A shard's part of a matrix, cut from the streaming layout on the device, equals the streaming layout of the same rows and
    columns cut from the GGUF tensor on the host, byte for byte (row padding included)."""
    from amd_c_b200 import kernels as K
    from amd_c_b200.backend import shard_cols

    rng = np.random.default_rng(rows * 7 + cols)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    whole = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    part = K.mat_part(whole, ranges, c0, c1 - c0)
    per_row = raw.reshape(rows, -1)
    sub = np.concatenate([shard_cols(per_row[r0: r0 + n].reshape(-1), typ, n, cols, c0, c1).reshape(n, -1) for r0, n in ranges])
    n_rows = sum(n for _, n in ranges)
    want = K.Mat.from_gguf(typ, dev(np.ascontiguousarray(sub).reshape(-1), cuda), n_rows, c1 - c0)
    assert part.rows == n_rows and part.cols == c1 - c0
    nbytes = lib.ie_b200_mat_bytes(part.kind, n_rows, c1 - c0)
    rowb = lib.ie_b200_row_bytes(part.kind, c1 - c0)
    used = {MAT_Q4: 18, MAT_Q8: 34, MAT_Q4K: 18, MAT_Q6K: 26, MAT_F32: 128}[part.kind] * ((c1 - c0) // 32) + (((c1 - c0) // 128) if part.kind == MAT_Q6K else 0)
    got_b, want_b = part.data.cpu().numpy()[:nbytes].reshape(n_rows, rowb), want.data.cpu().numpy()[:nbytes].reshape(n_rows, rowb)
    assert (got_b[:, :used] == want_b[:, :used]).all()
    assert (got_b[:, used:] == 0).all()


@pytest.mark.parametrize("typ,rows,cols", [(synth.GGML_Q4_0, 1000, 4096), (synth.GGML_Q4_0, 260, 14336), (synth.GGML_Q4_K, 520, 3584),
                                           (synth.GGML_Q6_K, 300, 3584), (synth.GGML_Q6_K, 64, 18944), (synth.GGML_Q4_K, 96, 5120),
                                           (synth.GGML_Q8_0, 700, 4096), (synth.GGML_Q8_0, 130, 14336)])
def test_gemv_model_shapes_with_epilogue(ora, cuda, typ, rows, cols):
    """Llama / Qwen column counts, rows not a multiple of the CTA tile, bias + residual, 3 tokens."""
    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows + cols)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    T = 3
    x = rng.standard_normal((T, cols)).astype(np.float32)
    bias = rng.standard_normal(rows).astype(np.float32)
    res = rng.standard_normal((T, rows)).astype(np.float32)
    xq = np.stack([ora.quant_q8(x[t]) for t in range(T)])
    y = K.gemv(m, dev(xq, cuda), bias=dev(bias, cuda), res=dev(res, cuda)).cpu().numpy()
    for t in range(T):
        want = ora.gemv(kind, qw, qs, rows, cols, xq[t], bias=bias, res=res[t])
        assert (bits(y[t]) == bits(want)).all(), t
    y0 = K.gemv(m, dev(xq[:1], cuda)).cpu().numpy()[0]
    assert (bits(y0) == bits(ora.gemv(kind, qw, qs, rows, cols, xq[0]))).all()


def test_gemv_linearity_full_size(ora, cuda):
    """At a full benchmark size (14336 x 4096) the oracle is too slow to sweep, so check properties: integer block
    dots are additive in the activations, and the GEMV of a zero activation is exactly zero."""
    import torch

    from amd_c_b200 import kernels as K

    rows, cols = 14336, 4096
    gen = torch.Generator(device=cuda).manual_seed(3)
    raw = synth.q4_0_normal_torch(gen, rows, cols, device=cuda)
    m = K.Mat.from_gguf(synth.GGML_Q4_0, raw.reshape(-1), rows, cols)
    rng = np.random.default_rng(0)
    nb = cols // 32
    qa = rng.integers(-60, 60, (2, cols)).astype(np.int8)

    def q8buf(q):
        b = np.zeros(40 * nb, np.uint8)
        b[: 32 * nb] = q.view(np.uint8)
        b[32 * nb: 36 * nb] = np.ones(nb, np.float32).view(np.uint8)
        b[36 * nb:] = q.reshape(nb, 32).astype(np.int64).sum(axis=1).astype(np.uint32).view(np.uint8)
        return b

    d0 = K.block_dots(m, dev(q8buf(qa[0]), cuda))
    d1 = K.block_dots(m, dev(q8buf(qa[1]), cuda))
    d01 = K.block_dots(m, dev(q8buf((qa[0].astype(np.int16) + qa[1]).astype(np.int8)), cuda))
    assert torch.equal(d0 + d1, d01)
    y = K.gemv(m, dev(np.zeros((1, 40 * nb), np.uint8), cuda))
    assert float(y.abs().max()) == 0.0
    # a sample of rows against the oracle, bit for bit
    sel = rng.choice(rows, 64, replace=False)
    sub = raw.reshape(rows, nb, 18)[torch.from_numpy(sel).to(cuda)].cpu().numpy()
    kind, qw, qs = ora.repack(synth.GGML_Q4_0, sub, 64, cols)
    xq = ora.quant_q8(rng.standard_normal(cols).astype(np.float32))
    yy = K.gemv(m, dev(xq, cuda).reshape(1, -1)).cpu().numpy()[0]
    assert (bits(yy[sel]) == bits(ora.gemv(kind, qw, qs, 64, cols, xq))).all()


def test_gemv_f32_bit_exact(ora, cuda):
    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(11)
    for rows, cols in [(1024, 256), (37, 100), (5, 4096), (3, 31)]:
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
        x = rng.standard_normal(cols).astype(np.float32)
        m = K.Mat(MAT_F32, rows, cols, dev(w, cuda))
        y = K.gemv(m, dev(x, cuda).reshape(1, -1)).cpu().numpy()[0]
        assert (bits(y) == bits(ora.gemv(MAT_F32, w, None, rows, cols, x))).all(), (rows, cols)


def test_embed_rmsnorm_swiglu_argmax(ora, cuda):
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(2)
    # embedding rows of a Q4_0 matrix: exact
    rows, cols = 300, 256
    raw = synth.make_gguf_bytes(synth.GGML_Q4_0, rng, rows, cols)
    kind, qw, qs = ora.repack(synth.GGML_Q4_0, raw, rows, cols)
    m = K.Mat.from_gguf(synth.GGML_Q4_0, dev(raw, cuda), rows, cols)
    toks = np.array([0, 299, 17], np.uint32)
    e = K.embed(m, dev(toks, cuda)).cpu().numpy()
    for i, t in enumerate(toks):
        assert (bits(e[i]) == bits(ora.embed_q4(qw, qs, cols // 32, int(t)))).all()
    # and of a Q8_0 matrix
    raw8 = synth.make_gguf_bytes(synth.GGML_Q8_0, rng, rows, cols)
    _, qw8, qs8 = ora.repack(synth.GGML_Q8_0, raw8, rows, cols)
    m8 = K.Mat.from_gguf(synth.GGML_Q8_0, dev(raw8, cuda), rows, cols)
    e8 = K.embed(m8, dev(toks, cuda)).cpu().numpy()
    for i, t in enumerate(toks):
        assert (bits(e8[i]) == bits(ora.embed_q8(qw8, qs8, cols // 32, int(t)))).all()
    # RMSNorm: tree sum vs sequential sum -> 1e-5 relative; the Q8 copy must be the quantiser of the kernel's own output
    for n in (256, 4096, 5120):
        x = rng.standard_normal((2, n)).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        y, q = K.rmsnorm(dev(x, cuda), dev(w, cuda), 1e-5)
        y, q = y.cpu().numpy(), q.cpu().numpy()
        for t in range(2):
            want = ora.rmsnorm(x[t], w, 1e-5)
            assert np.abs(y[t] - want).max() <= 1e-5 * np.abs(want).max()
            assert (q[t] == ora.quant_q8(y[t])).all()
    # SwiGLU: expf differs by an ulp or two from the host libm -> 1e-6 relative
    n = 14336
    gu = rng.standard_normal((2, 2 * n)).astype(np.float32) * 3
    d = dev(gu, cuda)
    a, q = K.swiglu(d, n)
    a, q = a.cpu().numpy(), q.cpu().numpy()
    for t in range(2):
        want = ora.swiglu(gu[t, :n], gu[t, n:])
        assert np.abs(a[t] - want).max() <= 1e-6 * np.abs(want).max()
        assert (q[t] == ora.quant_q8(a[t])).all()
    # argmax: first index among equal maxima
    x = rng.standard_normal((3, 128256)).astype(np.float32)
    x[1, 77] = x[1, 99000] = 50.0
    x[2, :] = 1.0
    out = K.argmax(dev(x, cuda)).cpu().numpy()
    for t in range(3):
        assert out[t, 0] == ora.argmax(x[t])
    p = out[:, 1].copy().view(np.float32)
    want_p = 1.0 / np.exp(x[0].astype(np.float64) - x[0].max()).sum()
    assert abs(p[0] - want_p) <= 1e-4 * want_p
    assert torch.cuda.is_available()


@pytest.mark.parametrize("n_head,n_kv,hd,neox,kv_f32", [(8, 4, 32, False, True), (8, 4, 32, False, False), (32, 8, 128, False, False),
                                                        (28, 4, 128, True, False), (40, 8, 128, True, True), (4, 4, 64, False, False),
                                                        (24, 8, 128, False, False), (12, 2, 64, True, False), (12, 2, 32, True, True)])
def test_rope_kv_and_attention(ora, cuda, n_head, n_kv, hd, neox, kv_f32):
    """RoPE + cache store is exact (f32 cache) or exact after half rounding; attention agrees with the oracle's
    two-pass softmax over the same cache within 1e-4 of the output scale, at positions that cross tile and split edges."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(n_head * 1000 + hd)
    n_ctx = 700
    cs, sn = ora.rope_tables(n_ctx, hd, 10000.0)
    qd, kvd = n_head * hd, n_kv * hd
    dt = torch.float32 if kv_f32 else torch.float16
    kc = torch.zeros((n_kv, n_ctx, hd), dtype=dt, device=cuda)
    vc = torch.zeros_like(kc)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(kc)  # the caches of the fused (RoPE + store + attention) kernel
    kc_ref, vc_ref = np.zeros((n_ctx, kvd), np.float32), np.zeros((n_ctx, kvd), np.float32)
    scratch = K.AttnScratch(n_head, hd, n_ctx, 1, cuda)
    d_cs, d_sn = dev(cs, cuda), dev(sn, cuda)
    check_at = {0, 1, 31, 63, 64, 65, 127, 128, 300, 511, 512, 699}
    # fill the cache in bulk for positions not checked one by one
    for pos in range(n_ctx):
        qkv = rng.standard_normal(qd + 2 * kvd).astype(np.float32)
        q_ref = ora.rope(qkv[:qd], n_head, hd, neox, cs[pos], sn[pos])
        k_ref = ora.rope(qkv[qd: qd + kvd], n_kv, hd, neox, cs[pos], sn[pos])
        v_ref = qkv[qd + kvd:]
        if not kv_f32:
            k_ref, v_ref = k_ref.astype(np.float16).astype(np.float32), v_ref.astype(np.float16).astype(np.float32)
        kc_ref[pos], vc_ref[pos] = k_ref, v_ref
        if pos in check_at:
            d = dev(qkv.reshape(1, -1), cuda)
            d_raw = d.clone()
            K.rope_kv(d, kc, vc, d_cs, d_sn, dev(np.array([pos], np.uint32), cuda), n_head, n_kv, hd, neox, n_ctx)
            got = d.cpu().numpy()[0]
            assert (bits(got[:qd]) == bits(q_ref)).all()
            assert (bits(kc[:, pos, :].float().cpu().numpy().reshape(-1)) == bits(k_ref)).all()
            assert (bits(vc[:, pos, :].float().cpu().numpy().reshape(-1)) == bits(v_ref)).all()
            out, oq = K.attn_decode(d, kc, vc, dev(np.array([pos], np.uint32), cuda), n_head, n_kv, hd, n_ctx, scratch)
            out, oq = out.cpu().numpy()[0], oq.cpu().numpy()[0]
            want = ora.attention(q_ref, kc_ref, vc_ref, pos, n_head, n_kv, hd)
            assert np.abs(out - want).max() <= 1e-4 * np.abs(want).max(), pos
            assert (oq == ora.quant_q8(out)).all(), pos
            assert int(scratch.count.abs().max()) == 0  # arrival counters are left at zero
            # the fused kernel: same cache rows bit for bit, same output as the two-kernel path to the last bit
            out2, oq2 = K.attn_decode_fused(d_raw, kc2, vc2, d_cs, d_sn, dev(np.array([pos], np.uint32), cuda), n_head, n_kv, hd, neox, n_ctx, scratch)
            assert torch.equal(kc2[:, pos, :], kc[:, pos, :]) and torch.equal(vc2[:, pos, :], vc[:, pos, :]), pos
            assert (bits(out2.cpu().numpy()[0]) == bits(out)).all(), pos
            assert (oq2.cpu().numpy()[0] == oq).all()
        else:
            kc[:, pos, :] = torch.from_numpy(k_ref.reshape(n_kv, hd)).to(cuda).to(dt)
            vc[:, pos, :] = torch.from_numpy(v_ref.reshape(n_kv, hd)).to(cuda).to(dt)
            kc2[:, pos, :], vc2[:, pos, :] = kc[:, pos, :], vc[:, pos, :]


def test_attention_multi_token_rows(ora, cuda):
    """T = 3 tokens in one launch: token t sees positions 0 .. pos + t (the chunk is causal)."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(8)
    n_head, n_kv, hd, n_ctx, T, pos0 = 8, 4, 32, 256, 3, 70
    kvd = n_kv * hd
    kc_ref = rng.standard_normal((n_ctx, kvd)).astype(np.float32)
    vc_ref = rng.standard_normal((n_ctx, kvd)).astype(np.float32)
    kc = torch.from_numpy(kc_ref.reshape(n_ctx, n_kv, hd).transpose(1, 0, 2).copy()).to(cuda)
    vc = torch.from_numpy(vc_ref.reshape(n_ctx, n_kv, hd).transpose(1, 0, 2).copy()).to(cuda)
    q = rng.standard_normal((T, n_head * hd)).astype(np.float32)
    scratch = K.AttnScratch(n_head, hd, n_ctx, T, cuda)
    out, _ = K.attn_decode(dev(q, cuda), kc, vc, dev(np.array([pos0], np.uint32), cuda), n_head, n_kv, hd, n_ctx, scratch)
    out = out.cpu().numpy()
    for t in range(T):
        want = ora.attention(q[t], kc_ref, vc_ref, pos0 + t, n_head, n_kv, hd)
        assert np.abs(out[t] - want).max() <= 1e-4 * np.abs(want).max(), t


@pytest.mark.parametrize("n_head,n_kv", [(32, 8), (40, 8), (24, 8)])
def test_attention_long_context(ora, cuda, n_head, n_kv):
    """Decode attention on the half cache at the context lengths the long-context benchmark runs at: with the real
    context size (32768) the launcher cuts the positions into up to 37 splits per KV head and picks the variant with
    3 tile buffers and two CTAs per SM; the merge of the splits' partials loops four splits at a time. Against the
    oracle's two-pass softmax over the same (half-rounded) cache, 1e-4 of the output scale; Q8 copy exact; the
    arrival counters back at zero. Also three tokens in one launch at 5000 positions."""
    import torch

    from amd_c_b200 import kernels as K

    hd, n_ctx = 128, 32768
    kvd = n_kv * hd
    gen = torch.Generator(device=cuda).manual_seed(n_head)
    kc = (torch.randn(n_kv, n_ctx, hd, device=cuda, generator=gen) * 0.7).half()
    vc = torch.randn(n_kv, n_ctx, hd, device=cuda, generator=gen).half()
    kc_ref = kc.float().permute(1, 0, 2).reshape(n_ctx, kvd).cpu().numpy()
    vc_ref = vc.float().permute(1, 0, 2).reshape(n_ctx, kvd).cpu().numpy()
    rng = np.random.default_rng(n_head)
    scratch = K.AttnScratch(n_head, hd, n_ctx, 3, cuda)
    for pos in (4095, 4096, 9000, 32767):
        q = rng.standard_normal((1, n_head * hd)).astype(np.float32)
        out, oq = K.attn_decode(dev(q, cuda), kc, vc, dev(np.array([pos], np.uint32), cuda), n_head, n_kv, hd, n_ctx, scratch)
        out, oq = out.cpu().numpy()[0], oq.cpu().numpy()[0]
        want = ora.attention(q[0], kc_ref, vc_ref, pos, n_head, n_kv, hd)
        assert np.abs(out - want).max() <= 1e-4 * np.abs(want).max(), pos
        assert (oq == ora.quant_q8(out)).all(), pos
        assert int(scratch.count.abs().max()) == 0, pos
    T, pos0 = 3, 5000
    q = rng.standard_normal((T, n_head * hd)).astype(np.float32)
    out, _ = K.attn_decode(dev(q, cuda), kc, vc, dev(np.array([pos0], np.uint32), cuda), n_head, n_kv, hd, n_ctx, scratch)
    out = out.cpu().numpy()
    for t in range(T):
        want = ora.attention(q[t], kc_ref, vc_ref, pos0 + t, n_head, n_kv, hd)
        assert np.abs(out[t] - want).max() <= 1e-4 * np.abs(want).max(), t
    assert int(scratch.count.abs().max()) == 0


def test_attention_long_context_fused_step(ora, cuda):
    """The one-token kernel with RoPE and the cache store folded in, at a long context (20000 positions, many splits):
    the split that owns the new position takes that row from registers. Same output as the oracle over the cache with
    the new (rotated, half-rounded) row in place, and the row is stored."""
    import torch

    from amd_c_b200 import kernels as K

    n_head, n_kv, hd, n_ctx, pos = 32, 8, 128, 32768, 20000
    qd, kvd = n_head * hd, n_kv * hd
    gen = torch.Generator(device=cuda).manual_seed(3)
    kc = (torch.randn(n_kv, n_ctx, hd, device=cuda, generator=gen) * 0.7).half()
    vc = torch.randn(n_kv, n_ctx, hd, device=cuda, generator=gen).half()
    cs, sn = ora.rope_tables(n_ctx, hd, 500000.0)
    rng = np.random.default_rng(3)
    qkv = rng.standard_normal(qd + 2 * kvd).astype(np.float32)
    scratch = K.AttnScratch(n_head, hd, n_ctx, 1, cuda)
    out, oq = K.attn_decode_fused(dev(qkv, cuda), kc, vc, dev(cs, cuda), dev(sn, cuda), dev(np.array([pos], np.uint32), cuda), n_head, n_kv, hd, False,
                                  n_ctx, scratch)
    q_ref = ora.rope(qkv[:qd], n_head, hd, False, cs[pos], sn[pos])
    k_ref = ora.rope(qkv[qd: qd + kvd], n_kv, hd, False, cs[pos], sn[pos]).astype(np.float16).astype(np.float32)
    v_ref = qkv[qd + kvd:].astype(np.float16).astype(np.float32)
    assert (bits(kc[:, pos, :].float().cpu().numpy().reshape(-1)) == bits(k_ref)).all()
    assert (bits(vc[:, pos, :].float().cpu().numpy().reshape(-1)) == bits(v_ref)).all()
    kc_ref = kc.float().permute(1, 0, 2).reshape(n_ctx, kvd).cpu().numpy()
    vc_ref = vc.float().permute(1, 0, 2).reshape(n_ctx, kvd).cpu().numpy()
    want = ora.attention(q_ref, kc_ref, vc_ref, pos, n_head, n_kv, hd)
    out = out.cpu().numpy()[0]
    assert np.abs(out - want).max() <= 1e-4 * np.abs(want).max()
    assert (oq.cpu().numpy()[0] == ora.quant_q8(out)).all()
    assert int(scratch.count.abs().max()) == 0


STREAM_SHAPES = [(synth.GGML_Q4_0, 1000, 4096), (synth.GGML_Q4_0, 260, 14336), (synth.GGML_Q4_0, 7, 96), (synth.GGML_Q4_0, 1536, 256),
                 (synth.GGML_Q4_0, 149, 1056), (synth.GGML_Q4_K, 520, 3584), (synth.GGML_Q6_K, 300, 3584), (synth.GGML_Q6_K, 64, 18944),
                 (synth.GGML_Q4_K, 333, 5120), (synth.GGML_Q4_0, 2, 16352), (synth.GGML_Q4_0, 4096, 14336), (synth.GGML_Q6_K, 3000, 18944),
                 (synth.GGML_Q4_0, 9000, 4096), (synth.GGML_Q4_K, 5000, 256), (synth.GGML_Q8_0, 1000, 4096), (synth.GGML_Q8_0, 7, 96),
                 (synth.GGML_Q8_0, 4096, 14336), (synth.GGML_Q8_0, 9000, 1056)]


@pytest.mark.parametrize("typ,rows,cols", STREAM_SHAPES)
def test_gemv_stream_bit_exact(ora, cuda, typ, rows, cols):
    """The decode GEMV (weights streamed into registers, programmatic dependent launch): same bits as the oracle, with
    bias and residual, for row counts below, at and above the warp count of the persistent grid, for short rows and for
    the long-row variant (one row per warp, 16 lane steps in flight)."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows * 7 + cols)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    bias = rng.standard_normal(rows).astype(np.float32)
    res = rng.standard_normal(rows).astype(np.float32)
    xq = ora.quant_q8(x)
    y = K.gemv_stream(m, dev(xq, cuda), bias=dev(bias, cuda), res=dev(res, cuda)).cpu().numpy()[0]
    assert (bits(y) == bits(ora.gemv(kind, qw, qs, rows, cols, xq, bias=bias, res=res))).all()
    y2 = K.gemv_stream(m, dev(xq, cuda)).cpu().numpy()[0]
    assert (bits(y2) == bits(ora.gemv(kind, qw, qs, rows, cols, xq))).all()
    # back-to-back launches on one stream (each may start before the previous one ends) still see finished inputs
    d_xq = dev(xq, cuda)
    ys = [K.gemv_stream(m, d_xq) for _ in range(4)]
    assert all(torch.equal(ys[0], t) for t in ys[1:])


@pytest.mark.parametrize("typ,rows,cols", [(synth.GGML_Q4_0, 6144, 4096), (synth.GGML_Q4_0, 1536, 256), (synth.GGML_Q4_K, 700, 3584),
                                           (synth.GGML_Q6_K, 512, 5120)])
def test_norm_gemv_stream(ora, cuda, typ, rows, cols):
    """RMSNorm + Q8 folded into the GEMV prologue: the normalised vector within 1e-5 of the oracle's sequential-sum
    norm; its Q8 copy is exactly the quantiser of that vector; the GEMV of it is bit-exact."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows + 3 * cols)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    res = rng.standard_normal(rows).astype(np.float32)
    y, xn, xq = K.norm_gemv_stream(m, dev(x, cuda), dev(nw, cuda), 1e-5, res=dev(res, cuda))
    y, xn, xq = y.cpu().numpy()[0], xn.cpu().numpy(), xq.cpu().numpy()
    want = ora.rmsnorm(x, nw, 1e-5)
    assert np.abs(xn - want).max() <= 1e-5 * np.abs(want).max()
    assert (xq == ora.quant_q8(xn)).all()
    assert (bits(y) == bits(ora.gemv(kind, qw, qs, rows, cols, xq, res=res))).all()
    # and the same vector as the stand-alone norm kernel
    yn, qn = K.rmsnorm(dev(x.reshape(1, -1), cuda), dev(nw, cuda), 1e-5)
    assert torch.equal(qn.reshape(-1).cpu(), torch.from_numpy(xq))


@pytest.mark.parametrize("typ,rows,cols", [(synth.GGML_Q4_0, 4096, 4096), (synth.GGML_Q4_0, 256, 768), (synth.GGML_Q6_K, 3584, 2048), (synth.GGML_Q4_0, 4096, 14336)])
def test_gemv_norm_tail(ora, cuda, lib, typ, rows, cols):
    """The GEMV whose last CTA normalises and quantises the finished result: y bit-exact, the norm within 1e-5 of
    the oracle's, its Q8 copy exactly the quantiser of that vector, the arrival counter back at zero; twice in a row."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows + cols)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    nw = (1 + 0.1 * rng.standard_normal(rows)).astype(np.float32)
    counter = torch.zeros(2, dtype=torch.int32, device=cuda)
    for rep in range(2):
        x = rng.standard_normal(cols).astype(np.float32)
        res = rng.standard_normal(rows).astype(np.float32)
        xq = ora.quant_q8(x)
        y = dev(res.copy(), cuda)  # in place: y = res + W x
        xn = torch.empty(rows, dtype=torch.float32, device=cuda)
        xnq = torch.empty(40 * (rows // 32), dtype=torch.uint8, device=cuda)
        d_xq, d_nw = dev(xq, cuda), dev(nw, cuda)  # named: a temporary would be freed (and its memory reused) before the kernel runs
        K.check(lib.ie_b200_gemv_norm_tail(m.kind, m.data.data_ptr(), rows, cols, d_xq.data_ptr(), y.data_ptr(), None, y.data_ptr(),
                                           d_nw.data_ptr(), 1e-5, xn.data_ptr(), xnq.data_ptr(), counter.data_ptr(), None))
        want_y = ora.gemv(kind, qw, qs, rows, cols, xq, res=res)
        assert (bits(y.cpu().numpy()) == bits(want_y)).all(), rep
        want_n = ora.rmsnorm(want_y, nw, 1e-5)
        got_n = xn.cpu().numpy()
        assert np.abs(got_n - want_n).max() <= 1e-5 * np.abs(want_n).max()
        assert (xnq.cpu().numpy() == ora.quant_q8(got_n)).all()
        assert int(counter.abs().max()) == 0


@pytest.mark.parametrize("n", [256, 4096, 8192])
def test_allreduce_norm_one_rank(ora, cuda, lib, n):
    """The tensor-parallel stop kernel with a world of one rank (no peer to wait for): x + part bit-exact, the norm
    within 1e-5 of the oracle's, its Q8 copy exactly the quantiser of that vector; the local-argmax exchange leaves
    (index + offset, probability) of the single slice. Two calls in a row (the slots alternate by parity)."""
    import ctypes as C

    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(n)
    h = C.c_void_p()
    K.check(lib.ie_b200_ar_create(0, 1, n, C.byref(h)))
    try:
        nw = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        d_nw, err = dev(nw, cuda), torch.zeros(1, dtype=torch.int32, device=cuda)
        for rep in range(2):
            x, part = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
            d_x, d_part = dev(x.copy(), cuda), dev(part, cuda)
            xn = torch.empty(n, dtype=torch.float32, device=cuda)
            xq = torch.empty(40 * (n // 32), dtype=torch.uint8, device=cuda)
            K.check(lib.ie_b200_ar_allreduce_norm(h, d_part.data_ptr(), d_x.data_ptr(), d_nw.data_ptr(), 1e-5, xn.data_ptr(), xq.data_ptr(), n,
                                                  err.data_ptr(), None))
            want_x = x + part
            assert (bits(d_x.cpu().numpy()) == bits(want_x)).all(), rep
            want_n, got_n = ora.rmsnorm(want_x, nw, 1e-5), xn.cpu().numpy()
            assert np.abs(got_n - want_n).max() <= 1e-5 * np.abs(want_n).max()
            assert (xq.cpu().numpy() == ora.quant_q8(got_n)).all()
            logits = dev(rng.standard_normal(n).astype(np.float32), cuda)
            res = torch.tensor([7, np.float32(0.25).view(np.int32)], dtype=torch.int32, device=cuda)
            K.check(lib.ie_b200_ar_argmax(h, logits.data_ptr(), res.data_ptr(), 1000, err.data_ptr(), None))
            got = res.cpu().numpy()
            assert int(got[0]) == 1007 and abs(float(got[1:2].view(np.float32)[0]) - 0.25) < 1e-6
        assert int(err.item()) == 0
    finally:
        lib.ie_b200_ar_destroy(h)


@pytest.mark.parametrize("typ,rows,cols", [(synth.GGML_Q4_0, 4096, 2048), (synth.GGML_Q4_0, 4096, 7168), (synth.GGML_Q6_K, 512, 1024)])
def test_gemv_allreduce_norm_one_rank(ora, cuda, lib, typ, rows, cols):
    """The K-split GEMV with the exchange folded in, in a world of one rank: part = W xq bit-exact, x + part bit-exact,
    the norm within 1e-5 of the oracle's and its Q8 copy exactly the quantiser of that vector; twice in a row."""
    import ctypes as C

    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows + cols)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    nw = (1 + 0.1 * rng.standard_normal(rows)).astype(np.float32)
    h = C.c_void_p()
    K.check(lib.ie_b200_ar_create(0, 1, rows, C.byref(h)))
    try:
        err, d_nw = torch.zeros(1, dtype=torch.int32, device=cuda), dev(nw, cuda)
        for rep in range(2):
            act, x = rng.standard_normal(cols).astype(np.float32), rng.standard_normal(rows).astype(np.float32)
            xq = ora.quant_q8(act)
            d_xq, d_x = dev(xq, cuda), dev(x.copy(), cuda)
            part = torch.empty(rows, dtype=torch.float32, device=cuda)
            xn = torch.empty(rows, dtype=torch.float32, device=cuda)
            xnq = torch.empty(40 * (rows // 32), dtype=torch.uint8, device=cuda)
            K.check(lib.ie_b200_gemv_allreduce_norm(h, m.kind, m.data.data_ptr(), rows, cols, d_xq.data_ptr(), part.data_ptr(), d_x.data_ptr(),
                                                    d_nw.data_ptr(), 1e-5, xn.data_ptr(), xnq.data_ptr(), err.data_ptr(), None))
            want_p = ora.gemv(kind, qw, qs, rows, cols, xq)
            assert (bits(part.cpu().numpy()) == bits(want_p)).all(), rep
            want_x = x + want_p
            assert (bits(d_x.cpu().numpy()) == bits(want_x)).all(), rep
            want_n, got_n = ora.rmsnorm(want_x, nw, 1e-5), xn.cpu().numpy()
            assert np.abs(got_n - want_n).max() <= 1e-5 * np.abs(want_n).max()
            assert (xnq.cpu().numpy() == ora.quant_q8(got_n)).all()
            assert int(err.item()) == 0
    finally:
        lib.ie_b200_ar_destroy(h)


@pytest.mark.parametrize("typ,rows,cols,T", [(synth.GGML_Q4_0, 256, 256, 17), (synth.GGML_Q4_0, 1000, 4096, 100), (synth.GGML_Q4_K, 3584, 3584, 256),
                                             (synth.GGML_Q6_K, 512, 1024, 131), (synth.GGML_Q4_K, 96, 512, 40),
                                             (synth.GGML_Q4_0, 77, 192, 33), (synth.GGML_Q4_0, 130, 320, 20)])
def test_gemm_matches_gemv(ora, cuda, typ, rows, cols, T):
    """The prompt-chunk GEMM (int8 tensor-core block dots, fp32 scaling in block order) against the multi-token GEMV,
    which is bit-exact with the CPU reference: equal to fp32 rounding (1e-5 of the largest output; the reference's own
    GEMM is "not bitwise" against its GEMV either), with bias and residual, ragged row and token counts. Rows that are
    not whole stages of 4 blocks (192 and 320 columns) take the kernel that reads its fragments from global memory."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows * 7 + cols + T)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    x = dev(rng.standard_normal((T, cols)).astype(np.float32), cuda)
    xq = K.quant_q8(x)
    bias = dev(rng.standard_normal(rows).astype(np.float32), cuda)
    res = dev(rng.standard_normal((T, rows)).astype(np.float32), cuda)
    want = K.gemv(m, xq, bias=bias, res=res).cpu().numpy()
    got = K.gemm(m, xq, bias=bias, res=res).cpu().numpy()
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    # one token of it against the oracle itself
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    t = T // 2
    ref = ora.gemv(kind, qw, qs, rows, cols, xq[t].cpu().numpy(), bias=bias.cpu().numpy(), res=res[t].cpu().numpy())
    assert np.abs(got[t] - ref).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("typ,rows,cols,T", [(synth.GGML_Q4_0, 256, 256, 17), (synth.GGML_Q4_0, 1000, 4096, 100), (synth.GGML_Q4_K, 3584, 3584, 256),
                                             (synth.GGML_Q6_K, 512, 1024, 131), (synth.GGML_Q4_K, 96, 512, 40), (synth.GGML_Q4_0, 77, 192, 33),
                                             (synth.GGML_Q4_0, 130, 320, 20), (synth.GGML_Q4_0, 5000, 4096, 300), (synth.GGML_Q6_K, 300, 18944, 64),
                                             (synth.GGML_Q4_K, 9000, 3584, 256), (synth.GGML_Q4_0, 1, 64, 1), (synth.GGML_Q8_0, 1000, 4096, 100),
                                             (synth.GGML_Q8_0, 77, 192, 33), (synth.GGML_Q8_0, 4096, 14336, 256)])
def test_gemm_tc_matches_gemv(ora, cuda, typ, rows, cols, T):
    """The prompt-chunk GEMM on tcgen05 / tensor memory (both operands as two half-precision terms, fp32 accumulation over the
    whole K in tensor memory) against the multi-token GEMV, which is bit-exact with the CPU reference: 1e-5 of the largest
    output, with bias and residual; ragged rows (the second 128-row tile partly or wholly empty), ragged tokens (N rounded up to
    16, more than one token tile), K split over several CTAs for matrices of few rows (partials added in split order)."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows * 7 + cols + T)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    x = dev((rng.standard_normal((T, cols)) * rng.choice([1e-3, 1.0, 40.0], size=(T, 1))).astype(np.float32), cuda)
    xq = K.quant_q8(x)
    bias = dev(rng.standard_normal(rows).astype(np.float32), cuda)
    res = dev(rng.standard_normal((T, rows)).astype(np.float32), cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    plain = K.gemv(m, xq).cpu().numpy()
    got0 = K.gemm_tc(m, xq, err=err).cpu().numpy()
    assert int(err.item()) == 0
    # every token row on its own scale (the rows differ by orders of magnitude)
    for t in range(T):
        assert np.abs(got0[t] - plain[t]).max() <= 1e-5 * np.abs(plain[t]).max(), t
    want = K.gemv(m, xq, bias=bias, res=res).cpu().numpy()
    got = K.gemm_tc(m, xq, bias=bias, res=res, err=err).cpu().numpy()
    assert int(err.item()) == 0
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    t = T // 2
    ref = ora.gemv(kind, qw, qs, rows, cols, xq[t].cpu().numpy())
    assert np.abs(got0[t] - ref).max() <= 1e-5 * np.abs(ref).max()


def test_gemm_tc_small_and_large_weights(ora, cuda):
    """Weights far below and above the half-precision sweet spot: the per-matrix power-of-two scale keeps the two-term split
    exact to 22 bits (Q4_0 scales of 2e-6 and of 300)."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(12)
    rows, cols, T = 300, 512, 40
    for sigma in (2e-6, 300.0):
        raw = synth.q4_0_normal(rng, rows, cols, sigma=sigma)
        m = K.Mat.from_gguf(synth.GGML_Q4_0, dev(raw, cuda), rows, cols)
        xq = K.quant_q8(dev(rng.standard_normal((T, cols)).astype(np.float32), cuda))
        want = K.gemv(m, xq).cpu().numpy()
        got = K.gemm_tc(m, xq).cpu().numpy()
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max(), sigma


@pytest.mark.parametrize("n_head,n_kv,hd,T,pos0", [(8, 2, 128, 9, 70), (28, 4, 128, 5, 200), (8, 8, 64, 19, 0), (10, 2, 64, 4, 129), (16, 2, 128, 3, 63),
                                                          (24, 8, 128, 11, 100), (12, 2, 64, 7, 300)])
def test_attention_prefill_chunk(ora, cuda, n_head, n_kv, hd, T, pos0):
    """A prompt chunk on the tensor cores (tokens of a KV head share passes over the half cache): every token against the
    oracle's two-pass softmax over the same (half-rounded) cache within 1e-4 of the output scale, the Q8 copies exactly the
    quantiser of the outputs; token counts that do not fill the last CTA, positions across tile edges, G = 1, 4, 5, 7, 8."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(n_head * 100 + T)
    n_ctx, kvd = pos0 + T + 5, n_kv * hd
    kc_ref = rng.standard_normal((n_ctx, kvd)).astype(np.float16).astype(np.float32)
    vc_ref = rng.standard_normal((n_ctx, kvd)).astype(np.float16).astype(np.float32)
    kc = torch.from_numpy(kc_ref.reshape(n_ctx, n_kv, hd).transpose(1, 0, 2).copy()).to(cuda).half()
    vc = torch.from_numpy(vc_ref.reshape(n_ctx, n_kv, hd).transpose(1, 0, 2).copy()).to(cuda).half()
    q = rng.standard_normal((T, n_head * hd)).astype(np.float32)
    out, oq = K.attn_prefill(dev(q, cuda), kc, vc, dev(np.array([pos0], np.uint32), cuda), n_head, n_kv, hd)
    out, oq = out.cpu().numpy(), oq.cpu().numpy()
    for t in range(T):
        want = ora.attention(q[t], kc_ref, vc_ref, pos0 + t, n_head, n_kv, hd)
        assert np.abs(out[t] - want).max() <= 1e-4 * np.abs(want).max(), t
        assert (oq[t] == ora.quant_q8(out[t])).all(), t


@pytest.mark.parametrize("typ,rows,cols,T", [(synth.GGML_Q4_0, 130, 1024, 11), (synth.GGML_Q4_K, 77, 512, 16), (synth.GGML_Q6_K, 40, 18944, 5),
                                             (synth.GGML_Q4_0, 9, 64, 2), (synth.GGML_Q8_0, 130, 1024, 11), (synth.GGML_Q8_0, 40, 4096, 16)])
def test_gemv_several_tokens_one_pass(ora, cuda, typ, rows, cols, T):
    """2..16 tokens share one pass over the weights (groups of 8 tokens per CTA, ragged last group): every token's row is
    bit for bit the oracle's one-token GEMV."""
    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(rows * 3 + T)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    kind, qw, qs = ora.repack(typ, raw, rows, cols)
    m = K.Mat.from_gguf(typ, dev(raw, cuda), rows, cols)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    res = rng.standard_normal((T, rows)).astype(np.float32)
    xq = np.stack([ora.quant_q8(x[t]) for t in range(T)])
    y = K.gemv(m, dev(xq, cuda), res=dev(res, cuda)).cpu().numpy()
    for t in range(T):
        assert (bits(y[t]) == bits(ora.gemv(kind, qw, qs, rows, cols, xq[t], res=res[t]))).all(), t


def test_allreduce_missing_rank_gives_up(cuda, lib):
    """Failure detection without a fault: a world of two ranks whose second rank never calls. The kernel's wait for
    the peer's words is bounded (2 s): it sets the device error word to 3 and returns, the context stays usable, and
    the next call on a complete world of one rank works."""
    import ctypes as C
    import time

    import torch

    from amd_c_b200 import kernels as K

    n = 256
    hs = (C.c_void_p * 2)()
    for r in range(2):
        h = C.c_void_p()
        K.check(lib.ie_b200_ar_create(r, 2, n, C.byref(h)))
        hs[r] = h
    try:
        for r in range(2):
            K.check(lib.ie_b200_ar_connect_local(hs[r], hs))
        x, part = torch.ones(n, device=cuda), torch.ones(n, device=cuda)
        nw, err = torch.ones(n, device=cuda), torch.zeros(1, dtype=torch.int32, device=cuda)
        xn, xq = torch.empty(n, device=cuda), torch.empty(40 * (n // 32), dtype=torch.uint8, device=cuda)
        t0 = time.time()
        K.check(lib.ie_b200_ar_allreduce_norm(hs[0], part.data_ptr(), x.data_ptr(), nw.data_ptr(), 1e-5, xn.data_ptr(), xq.data_ptr(), n,
                                              err.data_ptr(), None))
        torch.cuda.synchronize()
        waited = time.time() - t0
        assert int(err.item()) == 3
        assert 1.5 < waited < 10.0, waited
        # with the error word up, later stops of the same step do not wait again: each looks once and goes on
        t0 = time.time()
        for _ in range(3):
            K.check(lib.ie_b200_ar_allreduce_norm(hs[0], part.data_ptr(), x.data_ptr(), nw.data_ptr(), 1e-5, xn.data_ptr(), xq.data_ptr(), n,
                                                  err.data_ptr(), None))
            K.check(lib.ie_b200_ar_allreduce_add(hs[0], part.data_ptr(), x.data_ptr(), x.data_ptr(), n, err.data_ptr(), None))
        torch.cuda.synchronize()
        assert time.time() - t0 < 0.5 and int(err.item()) == 3
        # the context is intact: an ordinary kernel still runs and is right
        y = K.quant_q8(torch.full((1, 32), 2.0, device=cuda)).cpu().numpy()[0]
        assert (y[:32].view(np.int8) == 127).all()
    finally:
        for r in range(2):
            lib.ie_b200_ar_destroy(hs[r])


@pytest.mark.parametrize("world,typ,rows", [(2, synth.GGML_Q4_0, 512), (4, synth.GGML_Q4_0, 512), (8, synth.GGML_Q4_0, 512), (2, synth.GGML_Q4_K, 512),
                                            (4, synth.GGML_Q6_K, 512), (2, synth.GGML_Q8_0, 512),
                                            # rows of a real model: from four ranks up the reduction is a cluster of 8 CTAs (1, 2 and 3 passes)
                                            (2, synth.GGML_Q4_0, 4096), (4, synth.GGML_Q4_0, 5120), (8, synth.GGML_Q4_0, 4096), (8, synth.GGML_Q4_K, 12288)])
def test_tp_stop_ranks_in_order_bit_exact(ora, cuda, lib, world, typ, rows):
    """The tensor-parallel stop with real partners, the ranks of a world run one after the other on one GPU (their states
    connected in-process): every rank's K-split GEMV first (each stores its rows into the others' slots and waits for
    nobody), then every rank's reduction (all rows are there: no kernel waits for a later one). x + p_0 + p_1 + ... in rank
    order, bit for bit against the oracle's partial GEMVs added in that order on the host; the same bits on every rank;
    RMSNorm 1e-5 and its Q8 copy exact; twice, so that both slot parities and the epoch hand-over are used."""
    import ctypes as C

    import torch

    from amd_c_b200 import kernels as K
    from amd_c_b200.backend import shard_cols

    cols = 256 * world
    rng = np.random.default_rng(world)
    raw = synth.make_gguf_bytes(typ, rng, rows, cols)
    nw = (1 + 0.1 * rng.standard_normal(rows)).astype(np.float32)
    hs = (C.c_void_p * world)()
    for r in range(world):
        h = C.c_void_p()
        K.check(lib.ie_b200_ar_create(r, world, rows, C.byref(h)))
        hs[r] = h
    try:
        for r in range(world):
            K.check(lib.ie_b200_ar_connect_local(hs[r], hs))
        shards, mats = [], []
        for r in range(world):
            sub = np.ascontiguousarray(shard_cols(raw.reshape(-1), typ, rows, cols, r * 256, (r + 1) * 256)).reshape(-1)
            shards.append(ora.repack(typ, sub, rows, 256))
            mats.append(K.Mat.from_gguf(typ, dev(sub, cuda), rows, 256))
        d_nw = dev(nw, cuda)
        err = torch.zeros(1, dtype=torch.int32, device=cuda)
        x0 = rng.standard_normal(rows).astype(np.float32)
        d_x = [dev(x0.copy(), cuda) for _ in range(world)]
        want_x = x0.copy()
        for rep in range(2):
            act = rng.standard_normal(cols).astype(np.float32)
            xqs = [ora.quant_q8(act[r * 256: (r + 1) * 256]) for r in range(world)]
            d_xq = [dev(q, cuda) for q in xqs]
            part = [torch.empty(rows, dtype=torch.float32, device=cuda) for _ in range(world)]
            xn = [torch.empty(rows, dtype=torch.float32, device=cuda) for _ in range(world)]
            xnq = [torch.empty(40 * (rows // 32), dtype=torch.uint8, device=cuda) for _ in range(world)]
            for r in range(world):
                K.check(lib.ie_b200_gemv_push(hs[r], mats[r].kind, mats[r].data.data_ptr(), rows, 256, d_xq[r].data_ptr(), part[r].data_ptr(), None))
            for r in range(world):
                K.check(lib.ie_b200_ar_reduce_norm(hs[r], part[r].data_ptr(), d_x[r].data_ptr(), d_nw.data_ptr(), 1e-5, xn[r].data_ptr(),
                                                   xnq[r].data_ptr(), rows, err.data_ptr(), None))
            torch.cuda.synchronize()
            assert int(err.item()) == 0
            for r in range(world):
                kind, qw, qs = shards[r]
                p = ora.gemv(kind, qw, qs, rows, 256, xqs[r])
                assert (bits(part[r].cpu().numpy()) == bits(p)).all(), (rep, r)
                want_x = (want_x + p).astype(np.float32)
            for r in range(world):
                assert (bits(d_x[r].cpu().numpy()) == bits(want_x)).all(), (rep, r)
                got_n = xn[r].cpu().numpy()
                want_n = ora.rmsnorm(want_x, nw, 1e-5)
                assert np.abs(got_n - want_n).max() <= 1e-5 * np.abs(want_n).max()
                assert (xnq[r].cpu().numpy() == ora.quant_q8(got_n)).all()
    finally:
        for r in range(world):
            lib.ie_b200_ar_destroy(hs[r])


@pytest.mark.parametrize("n,K,T", [(1024, 1, 2), (1024, 40, 3), (128256, 64, 2), (152064, 50, 1), (5000, 64, 4), (70, 64, 1)])
def test_topk(cuda, n, K, T):
    """The K largest of each row, descending, equal values by rising index (what a stable sort of (-value, index) gives),
    with many exact ties in the rows (values rounded to a coarse grid) and -inf entries."""
    import torch

    from amd_c_b200 import kernels as K_

    rng = np.random.default_rng(n + K)
    x = np.round(rng.standard_normal((T, n)) * 8).astype(np.float32) / 8  # a coarse grid: thousands of equal values
    x[0, : min(n, 7)] = -np.inf
    val, idx = K_.topk(dev(x, cuda), K)
    val, idx = val.cpu().numpy(), idx.cpu().numpy()
    for t in range(T):
        order = np.lexsort((np.arange(n), -x[t]))[:K]
        assert (idx[t] == order).all(), t
        assert (val[t] == x[t][order]).all(), t


def test_topk_refuses_large_k(cuda, lib):
    import torch

    x = torch.zeros(1, 200000, device=cuda)
    out = torch.zeros(256, device=cuda)
    assert lib.ie_b200_topk(x.data_ptr(), 200000, 65, 1, 800000, out.data_ptr(), out.data_ptr(), out.data_ptr(), None) == -2
    assert lib.ie_b200_topk(x.data_ptr(), 200000, 64, 1, 800000, out.data_ptr(), out.data_ptr(), out.data_ptr(), None) == -2  # 98 slices x 64 candidates


@pytest.mark.parametrize("typ,ffn,dim", [(synth.GGML_Q4_0, 768, 256), (synth.GGML_Q4_0, 14336, 4096), (synth.GGML_Q4_K, 1024, 1024), (synth.GGML_Q6_K, 1792, 512)])
def test_swiglu_inside_the_gemvs(ora, cuda, lib, typ, ffn, dim):
    """SwiGLU moved into the GEMVs around it: the gate / up GEMV over interleaved rows writes silu(gate) * up itself, the GEMV
    after it quantises that vector in its prologue. Against the oracle's GEMV, SwiGLU, quantiser, GEMV: the two GEMVs bit for
    bit, the SwiGLU values within 1e-6 (expf), the Q8 copy exactly the quantiser of the values."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(ffn + dim)
    gate, up = synth.make_gguf_bytes(typ, rng, ffn, dim), synth.make_gguf_bytes(typ, rng, ffn, dim)
    down = synth.make_gguf_bytes(synth.GGML_Q4_0, rng, dim, ffn)
    mg, mu = K.Mat.from_gguf(typ, dev(gate, cuda), ffn, dim), K.Mat.from_gguf(typ, dev(up, cuda), ffn, dim)
    rowb = lib.ie_b200_row_bytes(mg.kind, dim)
    il = torch.stack((mg.data[: ffn * rowb].view(ffn, rowb), mu.data[: ffn * rowb].view(ffn, rowb)), dim=1).reshape(-1).contiguous()
    md = K.Mat.from_gguf(synth.GGML_Q4_0, dev(down, cuda), dim, ffn)
    x = rng.standard_normal(dim).astype(np.float32)
    xq = ora.quant_q8(x)
    d_xq = dev(xq, cuda)
    h = torch.empty(ffn, dtype=torch.float32, device=cuda)
    K.check(lib.ie_b200_gemv_swiglu(mg.kind, il.data_ptr(), 2 * ffn, dim, d_xq.data_ptr(), h.data_ptr(), None))
    kg, gw, gs = ora.repack(typ, gate, ffn, dim)
    ku, uw, us = ora.repack(typ, up, ffn, dim)
    g_ref, u_ref = ora.gemv(kg, gw, gs, ffn, dim, xq), ora.gemv(ku, uw, us, ffn, dim, xq)
    h_ref = ora.swiglu(g_ref, u_ref)
    got_h = h.cpu().numpy()
    assert np.abs(got_h - h_ref).max() <= 1e-6 * np.abs(h_ref).max()
    res = rng.standard_normal(dim).astype(np.float32)
    d_res = dev(res, cuda)
    hq = torch.empty(40 * (ffn // 32), dtype=torch.uint8, device=cuda)
    y = torch.empty(dim, dtype=torch.float32, device=cuda)
    K.check(lib.ie_b200_quant_gemv_stream(md.kind, md.data.data_ptr(), dim, ffn, h.data_ptr(), hq.data_ptr(), y.data_ptr(), None, d_res.data_ptr(), None))
    want_q = ora.quant_q8(got_h)
    assert (hq.cpu().numpy() == want_q).all()
    kd, dw, ds = ora.repack(synth.GGML_Q4_0, down, dim, ffn)
    assert (bits(y.cpu().numpy()) == bits(ora.gemv(kd, dw, ds, dim, ffn, want_q, res=res))).all()


def test_swiglu_interleaved_equals_planar(cuda, lib):
    """SwiGLU over interleaved (gate_i, up_i) pairs: the same bits as the planar kernel on the same values, outputs and Q8."""
    import torch

    from amd_c_b200 import kernels as K

    rng = np.random.default_rng(77)
    T, n = 3, 768
    g, u = rng.standard_normal((T, n)).astype(np.float32) * 3, rng.standard_normal((T, n)).astype(np.float32)
    planar = dev(np.concatenate([g, u], axis=1), cuda)
    want, want_q = K.swiglu(planar, n)
    il = dev(np.stack([g, u], axis=2).reshape(T, 2 * n), cuda)
    h = torch.empty((T, n), dtype=torch.float32, device=cuda)
    q = torch.empty((T, 40 * (n // 32)), dtype=torch.uint8, device=cuda)
    K.check(lib.ie_b200_swiglu_il(il.data_ptr(), h.data_ptr(), n, q.data_ptr(), T, 2 * n * 4, n * 4, 40 * (n // 32), None))
    assert torch.equal(h, want.contiguous()) and torch.equal(q, want_q)


def test_tp_group_refuses_one_gpu_twice(cuda, lib):
    """Shards whose kernels wait for one another must not share a GPU: the group refuses a device named twice, a device
    that does not exist, and more than eight ranks, before it allocates anything."""
    import ctypes as C

    grp = C.c_void_p()
    twice = (C.c_int * 2)(0, 0)
    assert lib.ie_b200_tp_group_create(2, twice, 1024, C.byref(grp)) < 0 and b"twice" in lib.ie_b200_last_error()
    missing = (C.c_int * 2)(0, 99)
    assert lib.ie_b200_tp_group_create(2, missing, 1024, C.byref(grp)) < 0
    assert lib.ie_b200_tp_group_create(9, None, 1024, C.byref(grp)) < 0
    assert not grp.value
