"""Build the test oracles.

  oracle/libie_oracle.so      the C restatement (ie_oracle.c), always
  oracle/_ref/libie_ref.so    the reference's own CPU sources compiled where
                              they lie (common.c gguf.c model.c plan.c cpu.c)
                              plus ref_shim.c, only when the reference tree
                              is present on this machine
  oracle/_ref/ie-run-cuda     the reference's ie-run host program linked with
                              this repository's src/cuda.c backend and
                              libie_b200.so, same condition

No reference source is copied: the compiler reads the files in place and
only the built objects land in oracle/_ref/ (git-ignored). Flags follow the
reference Makefile (-std=c11 -O2) with -ffp-contract=off stated explicitly,
so no product of two floats is ever fused with a following add.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
REF_OUT = HERE / "_ref"


def reference_dir() -> Path | None:
    """The reference checkout: $IE_REFERENCE_DIR, else a sibling directory
    named 'reference' next to the repository."""
    p = Path(os.environ.get("IE_REFERENCE_DIR", REPO.parent / "reference"))
    return p if (p / "src" / "cpu.c").is_file() else None


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("oracle build failed")


def _stale(out: Path, srcs: list[Path]) -> bool:
    if not out.is_file():
        return True
    t = out.stat().st_mtime
    return any(s.stat().st_mtime > t for s in srcs if s.exists())


CFLAGS = ["-std=c11", "-O2", "-ffp-contract=off", "-fPIC", "-D_GNU_SOURCE", "-w"]


def build_oracle(force: bool = False) -> Path:
    out = HERE / "libie_oracle.so"
    src = HERE / "ie_oracle.c"
    if force or _stale(out, [src]):
        _run(["gcc", *CFLAGS, "-shared", "-o", str(out), str(src), "-lm"])
    return out


def build_ref(force: bool = False) -> Path | None:
    """libie_ref.so from the reference's CPU sources; None if the tree is absent
    (then a previously built copy, if any, is used as it is)."""
    out = REF_OUT / "libie_ref.so"
    ref = reference_dir()
    if ref is None:
        return out if out.is_file() else None
    srcs = [ref / "src" / n for n in ("common.c", "gguf.c", "model.c", "plan.c", "cpu.c")]
    shim = HERE / "ref_shim.c"
    if force or _stale(out, srcs + [shim]):
        REF_OUT.mkdir(exist_ok=True)
        _run(["gcc", *CFLAGS, "-shared", "-I", str(ref / "src"), "-o", str(out), *map(str, srcs), str(shim), "-lm", "-ldl"])
    return out


def build_ie_run(force: bool = False) -> Path | None:
    """The reference's ie-run with src/cuda.c as its GPU backend. Needs the
    reference tree (for main.c, gen.c, model.c ...) and the built CUDA library."""
    out = REF_OUT / "ie-run-cuda"
    ref = reference_dir()
    lib = REPO / "amd_c_b200" / "libie_b200.so"
    cuda_c = REPO / "src" / "cuda.c"
    if ref is None or not cuda_c.is_file():
        return out if out.is_file() else None
    if not lib.is_file():
        return None
    srcs = [ref / "src" / n for n in ("common.c", "gguf.c", "model.c", "plan.c", "cpu.c", "gen.c", "main.c")]
    if force or _stale(out, srcs + [cuda_c, lib, REPO / "include" / "ie_b200.h"]):
        REF_OUT.mkdir(exist_ok=True)
        _run(["gcc", "-std=c11", "-O2", "-ffp-contract=off", "-D_GNU_SOURCE", "-w", "-I", str(ref / "src"), "-I", str(REPO / "include"),
              "-o", str(out), *map(str, srcs), str(cuda_c), "-L", str(lib.parent), "-lie_b200",
              "-Wl,-rpath,$ORIGIN/../../amd_c_b200", "-lm", "-ldl"])
    return out


def build_all(force: bool = False) -> None:
    build_oracle(force)
    build_ref(force)
    build_ie_run(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("oracle:", HERE / "libie_oracle.so")
    print("reference:", build_ref() or "absent")
    print("ie-run-cuda:", build_ie_run() or "absent")
