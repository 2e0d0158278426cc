"""Child process of test_switchable_variants: with whatever IE_B200_* switches the parent set, run the tiny models
and (1) assert the float-cache greedy ids against the golden ids of the reference CPU backend, (2) save the logits of the half-cache
run (a prompt of 40 as chunks of 32 + 8, then one step) to the .npz path given as the argument, for the parent to compare
across switches."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
from amd_c_b200 import gguf  # noqa: E402
from amd_c_b200.backend import Backend  # noqa: E402


def main():
    for name, fname, n_ctx in (("tiny", "tiny.npz", 512), ("tiny-k", "tiny_k.npz", 256), ("tiny-q8", "tiny_q8.npz", 256)):
        g = np.load(ROOT / "tests" / "golden" / fname)
        cfg = gguf.make_model(gguf.config(name), seed=int(g["seed"]))
        ids = [int(t) for t in g["ids"]]
        b = Backend(cfg, n_ctx, kv_f32=True)
        tok = ids[0]
        for pos in range(len(ids) - 1):
            nxt, _ = b.step(tok, pos)
            if pos + 1 >= 3:
                assert nxt == ids[pos + 1], f"{name}: greedy token differs from the reference CPU backend at position {pos}"
            tok = ids[pos + 1]
        b.close()
    rng = np.random.default_rng(11)
    out = {}
    for name in ("tiny", "tiny-k", "tiny-128", "tiny-q8"):
        cfg = gguf.make_model(gguf.config(name), seed=0)
        prompt = [int(t) for t in rng.integers(0, cfg.vocab, 40)]
        b = Backend(cfg, 96, T=32, kv_f32=False)
        b.run(0, prompt[:32], 0, last_only=True)
        first = int(b.run(0, prompt[32:], 32, last_only=True)[-1])
        lg0 = b.read_rows("logits", len(prompt) - 32 - 1, 1).view(np.float32)[0, : cfg.vocab].copy()
        lg1 = np.zeros(cfg.vocab, np.float32)
        nxt, _ = b.step(first, len(prompt), lg1)
        b.close()
        out[name + "_l0"], out[name + "_l1"], out[name + "_t"] = lg0, lg1, np.array([first, nxt])
    np.savez(sys.argv[1], **out)


if __name__ == "__main__":
    main()
