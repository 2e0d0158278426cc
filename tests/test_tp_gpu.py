"""Tensor-parallel decode on 2, 4 and 8 GPUs (skipped where fewer are visible): the sharded engines, in both step modes
(CUDA graph of one kernel per op with the one-kernel all-reduce + norm stop; persistent step kernel with the exchange
inside it), against the unsharded engine: logits of the first steps, identical tokens on every rank."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("world,mode,model", [(2, "graph", "tiny-tp"), (2, "kernel", "tiny-tp"), (2, "graph", "tiny-k"), (4, "graph", "tiny-tp"),
                                              (4, "kernel", "tiny-tp"), (8, "graph", "tiny-tp"), (8, "kernel", "tiny-tp")])
def test_tp_matches_single_gpu(cuda, world, mode, model):
    import torch

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port",
           str(29731 + world), str(ROOT / "tests" / "tp_worker.py"), mode, model]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    # a worker's own traceback sits far above the launcher's report: keep the lines that name it
    own = [ln for ln in r.stderr.splitlines() if "tp_worker.py" in ln or "Error" in ln or "assert" in ln]
    assert r.returncode == 0, r.stdout[-2000:] + "\n".join(own[:40]) + r.stderr[-1500:]
    assert "chained tokens identical" in r.stdout
    print(r.stdout[-300:])


@pytest.mark.parametrize("world,model", [(2, "tiny-tp"), (2, "tiny-k"), (2, "tiny-q8"), (4, "tiny-tp")])
def test_ie_run_drop_in_sharded(cuda, tmp_path, world, model):
    """The reference's own ie-run host program with src/cuda.c as its GPU backend and IE_TP=N: one process drives the N
    shards (matrix parts cut from the reference loader's arrays, one exchange behind every column-split GEMV). Against
    `--backend cpu`: the logits of the first positions, the greedy ids while the runs have not parted at a close call, the
    prompt as a chunk, and seeded sampling with the candidates merged from the ranks' top-K lists against the host's
    selection over the gathered logits."""
    import numpy as np
    import torch

    sys.path.insert(0, str(ROOT))
    from amd_c_b200 import gguf

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    exe = ROOT / "oracle" / "_ref" / "ie-run-cuda"
    if not exe.is_file():
        pytest.skip("oracle/_ref/ie-run-cuda not built (reference tree absent at build time)")
    cfg = gguf.make_model(gguf.config(model), seed=0)
    path = tmp_path / "m.gguf"
    gguf.write_gguf(path, cfg)
    env = {**os.environ, "IE_KV_F32": "1"}

    def run(*extra, tp=None, tokens="1,2,3,7,300,12"):
        e = dict(env)
        if tp:
            e["IE_TP"] = str(tp)
        r = subprocess.run([str(exe), str(path), "--tokens", tokens, "--n", "24", "--ctx", "64", *extra], capture_output=True, text=True,
                           timeout=300, env=e)
        assert r.returncode == 0, r.stderr[-2000:]
        if tp:
            assert f"cuda: {tp} GPUs" in r.stderr, r.stderr[-500:]
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("ids:")][0]
        return [int(t) for t in line.split()[1:]]

    def dump(p):
        rows = [ln.split() for ln in Path(p).read_text().splitlines()]
        return [(int(r[1]), np.array(r[2:], dtype=np.float32)) for r in rows]

    want = run("--backend", "cpu", "--dump-logits", str(tmp_path / "cpu.txt"))
    got = run("--backend", "gpu", "--dump-logits", str(tmp_path / "gpu.txt"), tp=world)
    lc, lg = dump(tmp_path / "cpu.txt"), dump(tmp_path / "gpu.txt")
    # The sharded sums add the ranks' partials in rank order (a different float order from one row sum): 1e-4 of the logit
    # scale until a Q8 rounding flips somewhere, a few 1e-3 .. 1e-2 after that; the runs may part at a close call.
    errs, same = [], 0
    for (tc, c), (tg, g) in zip(lc, lg):
        if tc != tg:
            break
        same += 1
        errs.append(float(np.abs(g - c).max() / np.abs(c).max()))
    print(f"ie-run cpu vs IE_TP={world} ({model}), relative logit error per position:", " ".join(f"{e:.1e}" for e in errs))
    if errs and errs[0] > 1e-4:  # where in the vocabulary the first position is off (one rank's slice? everything?)
        d0 = np.abs(lg[0][1] - lc[0][1])
        print("first position, max |diff| per vocabulary slice:", [float(x.max()) for x in np.array_split(d0, 2 * world)], "scale", float(np.abs(lc[0][1]).max()))
    assert errs and errs[0] <= 1e-4, errs
    assert max(errs) <= 3e-2, errs
    assert same >= 6 and got[:same] == want[:same]
    chunked = run("--backend", "gpu", "--chunk", "4", tp=world)  # the prompt in chunks of 4 through backend.run
    assert chunked[:7] == got[:7]
    # a prompt long enough for the tensor-core GEMM (20 tokens in one chunk: every stop of the chunk one exchange over 20 rows)
    long_prompt = ",".join(str((7 * i + 3) % 500) for i in range(20))
    by_steps = run("--backend", "gpu", "--dump-logits", str(tmp_path / "gpu20.txt"), tp=world, tokens=long_prompt)
    by_chunk = run("--backend", "gpu", "--chunk", "32", tp=world, tokens=long_prompt)
    assert by_chunk[:22] == by_steps[:22]
    sampled = run("--backend", "gpu", "--temp", "0.8", "--top-k", "40", "--seed", "3", tp=world)
    env["IE_HOST_TOPK"] = "1"
    sampled_host = run("--backend", "gpu", "--temp", "0.8", "--top-k", "40", "--seed", "3", tp=world)
    assert sampled == sampled_host and sampled != got


@pytest.mark.parametrize("world", [2, 4])
def test_one_thread_drives_the_shards(cuda, world):
    """ie_b200_tp_group: the shards of one model on `world` GPUs of THIS process, driven by one host thread (what src/cuda.c does
    under IE_TP): step with the gathered logits, a prompt chunk, and a device-chained decode run, against the unsharded engine
    on GPU 0. Every shard's work is enqueued before any shard is waited for; the ranks' tokens must agree (the group checks)."""
    import ctypes as C

    import numpy as np
    import torch

    sys.path.insert(0, str(ROOT))
    from amd_c_b200 import _lib, gguf
    from amd_c_b200._lib import check
    from amd_c_b200.backend import Backend

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    lib = _lib.load()
    cfg = gguf.make_model(gguf.config("tiny-tp"), seed=0)
    n_ctx, T = 160, 24
    grp = C.c_void_p()
    check(lib.ie_b200_tp_group_create(world, None, cfg.dim * T, C.byref(grp)))
    shards = []
    try:
        for r in range(world):
            check(lib.ie_b200_tp_group_use(grp, r))
            b = Backend(cfg, n_ctx, T=T, kv_f32=True, tp=world, rank=r, device=torch.device(f"cuda:{r}"))
            check(lib.ie_b200_tp_group_attach(grp, r, b.h, r * b.vocab_l, b.vocab_l))
            b.collective = True
            shards.append(b)
        single = Backend(cfg, n_ctx, T=T, kv_f32=True, device=torch.device("cuda:0"))
        got, want = np.zeros(cfg.vocab, np.float32), np.zeros(cfg.vocab, np.float32)
        nxt, ms = C.c_uint32(), C.c_double()
        tok, worst = 1, 0.0
        for pos in range(10):
            check(lib.ie_b200_tp_group_step(grp, tok, pos, got.ctypes.data_as(C.c_void_p), C.byref(nxt), C.byref(ms)))
            w_tok, _ = single.step(tok, pos, want)
            assert int(np.argmax(got)) == nxt.value
            worst = max(worst, float(np.abs(got - want).max() / np.abs(want).max()))
            tok = w_tok  # the unsharded engine leads
        assert worst <= 3e-2, worst
        # a prompt chunk over the same history on both sides
        chunk = ((np.arange(T, dtype=np.uint32) * 7 + 3) % cfg.vocab).astype(np.uint32)
        out = np.zeros(T, np.uint32)
        check(lib.ie_b200_tp_group_run(grp, chunk.ctypes.data_as(C.c_void_p), T, 10, 1, out.ctypes.data_as(C.c_void_p), None))
        w_out = single.run(0, chunk, 10, last_only=True)
        lg_w = np.ascontiguousarray(single.read_rows("logits", T - 1, 1)[0, : 4 * cfg.vocab]).view(np.float32)
        lg_g = np.concatenate([np.ascontiguousarray(s.read_rows("logits", T - 1, 1)[0, : 4 * s.vocab_l]).view(np.float32) for s in shards])
        d = float(np.abs(lg_g - lg_w).max() / np.abs(lg_w).max())
        assert d <= 3e-2, d
        top2 = np.sort(lg_w)[-2:]
        if top2[1] - top2[0] > 2 * float(np.abs(lg_g - lg_w).max()):
            assert int(out[-1]) == int(w_out[-1])
        # K tokens chained on the devices: the same on every rank (checked inside), and the unsharded engine's while no close call parts them
        K = 16
        dec = np.zeros(K, np.uint32)
        check(lib.ie_b200_tp_group_decode(grp, int(w_out[-1]), 10 + T, K, dec.ctypes.data_as(C.c_void_p), C.byref(ms)))
        w_dec, _ = single.decode(int(w_out[-1]), 10 + T, K)
        common = next((i for i, (a, b) in enumerate(zip(dec, w_dec)) if int(a) != int(b)), K)
        print(f"one thread, {world} shards: logits within {worst:.1e}, chunk within {d:.1e}, {common} of {K} chained tokens identical, {ms.value / K:.3f} ms per token")
        assert ms.value > 0
        single.close()
    finally:
        lib.ie_b200_tp_group_destroy(grp)
        for b in shards:
            b.collective = False
            b.close()
