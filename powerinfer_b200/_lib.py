"""ctypes binding of libpowerinfer_b200.so (the C ABI declared in include/powerinfer_b200.h).

There is no fallback: if the library is missing the import fails, and every call that returns a
non-zero status raises with the library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libpowerinfer_b200.so")

PI_TYPE_F16, PI_TYPE_Q4_0 = 1, 2


class PiError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} not built: run `python -m powerinfer_b200.build` (needs nvcc)")
    lib = C.CDLL(LIB_PATH)
    vp, i64, i32, f32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t
    sig = {
        "pi_last_error": (C.c_char_p, []),
        "pi_version": (i32, []),
        "pi_row_bytes": (sz, [i32, i64]),
        "pi_workspace_bytes": (sz, [i64, i64, i32]),
        "pi_quantize_q4_0": (i32, [vp, vp, i64, i64, vp]),
        "pi_q4_0_repack": (i32, [vp, vp, i64, i64, vp]),
        "pi_dequantize_q4_0": (i32, [vp, vp, i64, i64, vp]),
        "pi_quantize_q8_0": (i32, [vp, vp, i64, i64, vp]),
        "pi_mul_mat_idx": (i32, [i32, vp, i64, i64, vp, i32, vp, i64, vp, f32, vp, i64, vp, sz, vp]),
        "pi_axpy": (i32, [i32, vp, i64, i64, vp, i32, i64, vp, i64, vp, f32, vp, vp, sz, vp]),
        "pi_sparse_ffn": (i32, [i32, vp, vp, vp, i64, i64, vp, i32, vp, i64, vp, f32, vp, vp, vp, sz, vp]),
        "pi_axpy_static_max_bytes": (sz, []),
        "pi_axpy_static": (i32, [i32, vp, i64, i64, vp, i64, vp, i64, vp, f32, vp, vp]),
        "pi_op_status": (i32, [vp, vp]),
        "pi_mul_mat": (i32, [i32, vp, i64, i64, vp, i32, vp, vp, vp, sz, vp]),
        "pi_predictor": (i32, [vp, vp, i64, i64, i64, vp, i32, vp, vp, sz, vp]),
        "pi_active_list": (i32, [vp, i64, i32, i64, f32, vp, vp, vp, sz, vp]),
        "pi_norm": (i32, [vp, i32, i64, i32, f32, vp, vp, vp, vp]),
        "pi_rope": (i32, [vp, i32, i32, i32, vp, vp, i32, vp]),
        "pi_rope_table_host": (None, [vp, i32, i32, f32]),
        "pi_attention_decode": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()
EXPORTS = ["pi_last_error", "pi_version", "pi_row_bytes", "pi_workspace_bytes", "pi_quantize_q4_0", "pi_q4_0_repack",
           "pi_dequantize_q4_0", "pi_quantize_q8_0", "pi_mul_mat_idx", "pi_axpy", "pi_sparse_ffn", "pi_axpy_static_max_bytes", "pi_axpy_static", "pi_op_status",
           "pi_mul_mat", "pi_predictor",
           "pi_active_list", "pi_norm", "pi_rope", "pi_rope_table_host", "pi_attention_decode"]


def check(rc: int) -> None:
    if rc != 0:
        raise PiError(f"powerinfer_b200 error {rc}: {lib.pi_last_error().decode("utf-8", errors="replace")}")
