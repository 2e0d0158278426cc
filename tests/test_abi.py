"""The C ABI: the library loads, exports every symbol the headers declare, and
refuses bad arguments with a message instead of launching (no GPU needed)."""
import ctypes
import re
from pathlib import Path

from amd_c_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"\b(ie_b200_\w+)\s*\(", h.read_text()))
    return names


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported by libie_b200.so"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"


def test_layout_sizes(lib):
    assert lib.ie_b200_row_bytes(_lib.MAT_Q4, 4096) == 128 * 18
    assert lib.ie_b200_row_bytes(_lib.MAT_Q4, 96) == 64  # 3 blocks: 54 bytes rounded up to 16
    assert lib.ie_b200_row_bytes(_lib.MAT_Q4K, 3584) == 112 * 18
    assert lib.ie_b200_row_bytes(_lib.MAT_Q6K, 256) == 224  # 210 rounded up
    assert lib.ie_b200_mat_bytes(_lib.MAT_F32, 3, 5) == 60
    assert lib.ie_b200_mat_bytes(_lib.MAT_Q4, 128256, 4096) == 128256 * 2304


def test_bad_arguments_are_refused(lib):
    assert lib.ie_b200_gemv(_lib.MAT_Q4, None, 8, 64, None, None, None, None, 1, 0, 0, 0, None) == -1
    assert b"NULL" in lib.ie_b200_last_error()
    buf = ctypes.create_string_buffer(4096)
    p = (ctypes.addressof(buf) + 15) & ~15
    assert lib.ie_b200_gemv(_lib.MAT_Q4, p, 8, 48, p, p, None, None, 1, 0, 0, 0, None) == -2  # cols not a multiple of 32
    assert lib.ie_b200_gemv(99, p, 8, 64, p, p, None, None, 1, 0, 0, 0, None) == -1
    assert lib.ie_b200_gemv(_lib.MAT_Q4K, p, 8, 64, p, p, None, None, 1, 0, 0, 0, None) == -2  # K kinds need cols % 256 == 0
    assert lib.ie_b200_attn_decode(p, p, p, p, None, p, 8, 3, 32, 0, 64, 64, 1, 0, 0, 0, p, p, None) == -2  # 8 heads over 3 KV heads
