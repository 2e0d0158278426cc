"""ctypes binding of libie_b200.so (the C ABI of include/ie_b200.h).

The library is the only compute path of this package: if it is missing or a
call fails, an exception is raised; nothing falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libie_b200.so"

MAT_Q4, MAT_F32, MAT_Q8, MAT_Q4K, MAT_Q6K = 0, 1, 2, 3, 4
GGML_F32, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 0, 2, 8, 12, 14
GGML_TO_MAT = {GGML_F32: MAT_F32, GGML_Q4_0: MAT_Q4, GGML_Q8_0: MAT_Q8, GGML_Q4_K: MAT_Q4K, GGML_Q6_K: MAT_Q6K}

_vp, _u32, _sz, _int, _f32 = C.c_void_p, C.c_uint32, C.c_size_t, C.c_int, C.c_float

# name -> (restype, argtypes); every symbol include/ie_b200.h declares
SIGNATURES = {
    "ie_b200_last_error": (C.c_char_p, []),
    "ie_b200_device_count": (_int, []),
    "ie_b200_launch_count": (C.c_uint64, []),
    "ie_b200_row_bytes": (_sz, [_int, _u32]),
    "ie_b200_mat_bytes": (_sz, [_int, _u32, _u32]),
    "ie_b200_repack_gguf": (_int, [_int, _vp, _u32, _u32, _vp, _vp]),
    "ie_b200_repack_ref": (_int, [_int, _vp, _vp, _u32, _u32, _vp, _vp]),
    "ie_b200_mat_part": (_int, [_int, _vp, _u32, _u32, _u32, _vp, _vp, _u32, _u32, _vp, _vp]),
    "ie_b200_quant_q8": (_int, [_vp, _vp, _u32, _u32, _sz, _sz, _vp]),
    "ie_b200_gemv": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _u32, _sz, _sz, _sz, _vp]),
    "ie_b200_gemm": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _u32, _sz, _sz, _sz, _vp]),
    "ie_b200_gemm_tc_scratch_bytes": (_sz, [_u32, _u32, _u32]),
    "ie_b200_mat_tc_exp": (_int, [_int, _vp, _u32, _u32, C.POINTER(_int), _vp]),
    "ie_b200_gemm_tc": (_int, [_int, _vp, _u32, _u32, _int, _vp, _vp, _vp, _vp, _u32, _sz, _sz, _sz, _vp, _sz, _vp, _vp]),
    "ie_b200_gemv_stream": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "ie_b200_norm_gemv_stream": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ie_b200_gemv_swiglu": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _vp]),
    "ie_b200_quant_gemv_stream": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ie_b200_gemv_norm_tail": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp]),
    "ie_b200_block_dots": (_int, [_int, _vp, _u32, _u32, _vp, _vp, _vp]),
    "ie_b200_embed": (_int, [_int, _vp, _u32, _vp, _vp, _u32, _sz, _vp]),
    "ie_b200_rmsnorm": (_int, [_vp, _vp, _vp, _u32, _f32, _vp, _u32, _sz, _sz, _sz, _vp]),
    "ie_b200_swiglu": (_int, [_vp, _vp, _u32, _vp, _u32, _sz, _sz, _vp]),
    "ie_b200_swiglu_il": (_int, [_vp, _vp, _u32, _vp, _u32, _sz, _sz, _sz, _vp]),
    "ie_b200_rope_kv": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _int, _int, _u32, _u32, _sz, _vp]),
    "ie_b200_attn_part_bytes": (_sz, [_u32, _u32, _u32, _u32]),
    "ie_b200_attn_count_words": (_sz, [_u32, _u32]),
    "ie_b200_attn_decode": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _int, _u32, _u32, _u32, _sz, _sz, _sz, _vp, _vp, _vp]),
    "ie_b200_attn_decode_fused": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _int, _int, _u32, _u32, _vp, _vp, _vp]),
    "ie_b200_attn_persistent_scratch_bytes": (_sz, [_u32, _u32, _u32]),
    "ie_b200_attn_persistent": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _int, _u32, _vp, _vp, _vp]),
    "ie_b200_attn_prefill": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _sz, _sz, _sz, _vp]),
    "ie_b200_argmax_part_bytes": (_sz, [_u32]),
    "ie_b200_argmax": (_int, [_vp, _u32, _vp, _u32, _sz, _sz, _vp, _vp]),
    "ie_b200_topk_scratch_bytes": (_sz, [_u32, _u32, _u32]),
    "ie_b200_topk": (_int, [_vp, _u32, _u32, _u32, _sz, _vp, _vp, _vp, _vp]),
    "ie_b200_argmax_static_max_rows": (_u32, []),
    "ie_b200_argmax_static": (_int, [_vp, _u32, _vp, _u32, _sz, _sz, _vp]),
}


# ---- the engine ABI (include/ie_b200_engine.h) ----
class Op(C.Structure):
    _fields_ = [("kind", C.c_int32), ("mat", C.c_int32), ("vec", C.c_int32), ("layer", C.c_int32), ("n", C.c_uint32), ("nh", C.c_uint32),
                ("a", C.c_uint64), ("b", C.c_uint64), ("c", C.c_uint64), ("qo", C.c_uint64), ("res", C.c_uint64),
                ("a_stride", C.c_uint32), ("b_stride", C.c_uint32), ("c_stride", C.c_uint32), ("qo_stride", C.c_uint32),
                ("res_stride", C.c_uint32)]


class EngineDesc(C.Structure):
    _fields_ = [("n_head", C.c_uint32), ("n_kv", C.c_uint32), ("hd", C.c_uint32), ("n_ctx", C.c_uint32), ("n_kv_layers", C.c_uint32),
                ("T_max", C.c_uint32), ("vocab", C.c_uint32), ("eps", C.c_float), ("neox", C.c_int32), ("kv_f32", C.c_int32),
                ("arena_bytes", C.c_uint64), ("logits_off", C.c_uint64), ("argmax_off", C.c_uint64), ("logits_stride", C.c_uint32),
                ("argmax_stride", C.c_uint32)]


_u64 = C.c_uint64
ENGINE_SIGNATURES = {
    "ie_b200_engine_create": (_int, [C.POINTER(EngineDesc), C.POINTER(_vp)]),
    "ie_b200_engine_destroy": (None, [_vp]),
    "ie_b200_engine_add_mat_gguf": (_int, [_vp, _int, _u32, _u32, _vp]),
    "ie_b200_engine_add_mat_ref": (_int, [_vp, _int, _u32, _u32, _vp, _vp]),
    "ie_b200_engine_add_mat_ref_part": (_int, [_vp, _int, _u32, _u32, _vp, _vp, _u32, _vp, _vp, _u32, _u32]),
    "ie_b200_engine_add_mat_device": (_int, [_vp, _int, _u32, _u32, _vp]),
    "ie_b200_engine_add_vec": (_int, [_vp, _vp, _u32]),
    "ie_b200_engine_set_rope": (_int, [_vp, _vp, _vp]),
    "ie_b200_engine_set_ops": (_int, [_vp, C.POINTER(Op), _u32, _u32]),
    "ie_b200_engine_step": (_int, [_vp, _u32, _u32, _vp, C.POINTER(_u32), C.POINTER(C.c_double)]),
    "ie_b200_engine_clear_error": (_int, [_vp]),
    "ie_b200_engine_set_step_mode": (_int, [_vp, _int]),
    "ie_b200_engine_step_is_kernel": (_int, [_vp]),
    "ie_b200_engine_inject_abort": (_int, [_vp]),
    "ie_b200_engine_phase_times": (_int, [_vp, _int, _vp]),
    "ie_b200_engine_decode": (_int, [_vp, _u32, _u32, _u32, _vp, C.POINTER(C.c_double)]),
    "ie_b200_engine_enqueue_kinds": (_int, [_vp, _u32, _u32, _u32, _u32, _vp]),
    "ie_b200_engine_run": (_int, [_vp, _vp, _u32, _u32, _int, _vp, _vp]),
    "ie_b200_engine_step_begin": (_int, [_vp, _u32, _u32, _int]),
    "ie_b200_engine_step_end": (_int, [_vp, _vp, C.POINTER(_u32), C.POINTER(C.c_double)]),
    "ie_b200_engine_decode_begin": (_int, [_vp, _u32, _u32, _u32]),
    "ie_b200_engine_decode_end": (_int, [_vp, _vp, C.POINTER(C.c_double)]),
    "ie_b200_engine_run_begin": (_int, [_vp, _vp, _u32, _u32, _int]),
    "ie_b200_engine_run_end": (_int, [_vp, _vp, _vp]),
    "ie_b200_engine_read_rows": (_int, [_vp, _u64, _u32, _u32, _u32, _vp]),
    "ie_b200_engine_copy_rows": (_int, [_vp, _u64, _u32, _u32, _u64, _u32, _u32, _u32, _u32, _int]),
    "ie_b200_engine_topk": (_int, [_vp, _u64, _u32, _u32, _u32, _u32, _u32, _vp, _vp]),
    "ie_b200_engine_write_rows": (_int, [_vp, _u64, _u32, _u32, _u32, _vp]),
    "ie_b200_engine_set_collective": (_int, [_vp, _vp, _u32]),
    "ie_b200_engine_set_input": (_int, [_vp, _vp, _u32, _u32, _vp]),
    "ie_b200_engine_enqueue": (_int, [_vp, _u32, _u32, _u32, _vp]),
    "ie_b200_engine_arena": (_vp, [_vp]),
    "ie_b200_engine_input_scalars": (_vp, [_vp]),
    "ie_b200_engine_weight_bytes_per_token": (_u64, [_vp]),
    "ie_b200_engine_launches_per_step": (_u32, [_vp]),
}


SIGNATURES.update(ENGINE_SIGNATURES)

# ---- the tensor-parallel all-reduce (include/ie_b200_tp.h) ----
SIGNATURES.update({
    "ie_b200_ar_create": (_int, [_u32, _u32, _u32, C.POINTER(_vp)]),
    "ie_b200_ar_handles": (_int, [_vp, _vp]),
    "ie_b200_ar_connect": (_int, [_vp, _vp]),
    "ie_b200_ar_connect_local": (_int, [_vp, C.POINTER(_vp)]),
    "ie_b200_ar_allreduce_add": (_int, [_vp, _vp, _vp, _vp, _u32, _vp, _vp]),
    "ie_b200_ar_allreduce_norm": (_int, [_vp, _vp, _vp, _vp, _f32, _vp, _vp, _u32, _vp, _vp]),
    "ie_b200_gemv_allreduce_norm": (_int, [_vp, _int, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp]),
    "ie_b200_gemv_push": (_int, [_vp, _int, _vp, _u32, _u32, _vp, _vp, _vp]),
    "ie_b200_ar_reduce_norm": (_int, [_vp, _vp, _vp, _vp, _f32, _vp, _vp, _u32, _vp, _vp]),
    "ie_b200_ar_argmax": (_int, [_vp, _vp, _vp, _u32, _vp, _vp]),
    "ie_b200_ar_destroy": (None, [_vp]),
    "ie_b200_tp_group_create": (_int, [_u32, _vp, _u32, C.POINTER(_vp)]),
    "ie_b200_tp_group_use": (_int, [_vp, _u32]),
    "ie_b200_tp_group_attach": (_int, [_vp, _u32, _vp, _u32, _u32]),
    "ie_b200_tp_group_step": (_int, [_vp, _u32, _u32, _vp, C.POINTER(_u32), C.POINTER(C.c_double)]),
    "ie_b200_tp_group_run": (_int, [_vp, _vp, _u32, _u32, _int, _vp, _vp]),
    "ie_b200_tp_group_decode": (_int, [_vp, _u32, _u32, _u32, _vp, C.POINTER(C.c_double)]),
    "ie_b200_tp_group_destroy": (None, [_vp]),
})


class IeB200Error(RuntimeError):
    """A call into libie_b200.so returned a negative status."""


_lib = None


def load() -> C.CDLL:
    """Load the library (once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.is_file():
            raise IeB200Error(f"{LIB_PATH} is missing: run `python -m amd_c_b200.build` (needs nvcc); there is no CPU fallback")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = load().ie_b200_last_error().decode("utf-8", "replace")
        raise IeB200Error(f"libie_b200 status {status}: {msg}")


def require_gpu() -> None:
    if load().ie_b200_device_count() < 1:
        raise IeB200Error("no CUDA device: the amd_c_b200 kernels need a GPU (there is no CPU fallback)")
