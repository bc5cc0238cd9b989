"""ctypes binding of ``libaf3k.so`` (the C ABI declared in ``include/af3k.h``).

This module is the only place that touches the shared library.  It never falls back to a
CPU or PyTorch implementation: when the library is missing, or a call returns an error
code, it raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
# AF3K_LIBRARY points at another build of the same library (kernel experiments)
LIB_PATH = os.environ.get("AF3K_LIBRARY") or os.path.join(_HERE, "libaf3k.so")

AF3K_BF16, AF3K_F32, AF3K_FP8_E4M3 = 0, 1, 2
AF3K_STATUS_WAIT_TIMEOUT = 1

# every symbol include/af3k.h declares
EXPORTED_SYMBOLS = (
    "af3k_version",
    "af3k_strerror",
    "af3k_last_error_detail",
    "af3k_dot_product_attention_workspace",
    "af3k_stage_bias",
    "af3k_dot_product_attention",
    "af3k_dot_product_attention_noalloc",
    "af3k_static_scratch_bytes",
    "af3k_last_launch_count",
    "af3k_set_wait_limit_cycles",
    "af3k_describe_plan",
    "af3k_pair_bias_status",
    "af3k_pair_front",
    "af3k_debug_set_dump",
    "af3k_selftest_wait_timeout",
    "af3k_pair_bias",
    "af3k_sigmoid_gate",
    "af3k_qkvg_projection",
)


class AttentionDesc(ctypes.Structure):
    """Mirror of ``af3k_attention_desc``."""

    _fields_ = [
        ("B1", ctypes.c_int64),
        ("B2", ctypes.c_int64),
        ("Sq", ctypes.c_int64),
        ("Sk", ctypes.c_int64),
        ("D", ctypes.c_int64),
        ("q_stride", ctypes.c_int64 * 3),
        ("k_stride", ctypes.c_int64 * 3),
        ("v_stride", ctypes.c_int64 * 3),
        ("out_stride", ctypes.c_int64 * 3),
        ("bias_stride", ctypes.c_int64 * 2),
        ("mask_row_stride", ctypes.c_int64),
        ("qk_dtype", ctypes.c_int32),
        ("bias_dtype", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("rows_per_item", ctypes.c_int32),
        ("bias_prescaled", ctypes.c_int32),
        ("max_ctas", ctypes.c_int32),
    ]


class Af3kError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"libaf3k error {code}: {text}")
        self.code = code


_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Loads libaf3k.so once and sets the prototypes.  Raises if the library was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m af3_kernels_b200.build` "
            "(nvcc, sm_100a).  There is no CPU fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, sz = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_size_t
    dp = ctypes.POINTER(AttentionDesc)
    lib.af3k_version.restype = ctypes.c_int
    lib.af3k_version.argtypes = []
    lib.af3k_strerror.restype = ctypes.c_char_p
    lib.af3k_strerror.argtypes = [ctypes.c_int]
    lib.af3k_last_error_detail.restype = ctypes.c_char_p
    lib.af3k_last_error_detail.argtypes = []
    lib.af3k_dot_product_attention_workspace.restype = sz
    lib.af3k_dot_product_attention_workspace.argtypes = [dp, vp]
    lib.af3k_stage_bias.restype = ctypes.c_int
    lib.af3k_stage_bias.argtypes = [dp, vp, vp, vp, vp, sz, vp]
    lib.af3k_dot_product_attention.restype = ctypes.c_int
    lib.af3k_dot_product_attention.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp, vp]
    lib.af3k_dot_product_attention_noalloc.restype = ctypes.c_int
    lib.af3k_dot_product_attention_noalloc.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.af3k_static_scratch_bytes.restype = sz
    lib.af3k_static_scratch_bytes.argtypes = []
    lib.af3k_last_launch_count.restype = ctypes.c_int
    lib.af3k_last_launch_count.argtypes = []
    lib.af3k_set_wait_limit_cycles.restype = None
    lib.af3k_set_wait_limit_cycles.argtypes = [i64]
    lib.af3k_describe_plan.restype = ctypes.c_int
    lib.af3k_describe_plan.argtypes = [dp, ctypes.POINTER(ctypes.c_int32)]
    lib.af3k_debug_set_dump.restype = None
    lib.af3k_debug_set_dump.argtypes = [vp]
    lib.af3k_selftest_wait_timeout.restype = ctypes.c_int
    lib.af3k_selftest_wait_timeout.argtypes = [i64, vp, vp]
    lib.af3k_pair_bias.restype = ctypes.c_int
    lib.af3k_pair_bias.argtypes = [vp, ctypes.c_int32, i64, i64, i64, i64, vp, vp, vp, ctypes.c_float, vp, vp,
                                   i64, vp]
    lib.af3k_pair_bias_status.restype = ctypes.c_int
    lib.af3k_pair_bias_status.argtypes = [ctypes.POINTER(ctypes.c_int32)]
    lib.af3k_qkvg_projection.restype = ctypes.c_int
    lib.af3k_qkvg_projection.argtypes = [vp, vp, i64, i64, i64, ctypes.c_float, vp, vp, vp, vp, vp, vp]
    lib.af3k_pair_front.restype = ctypes.c_int
    lib.af3k_pair_front.argtypes = [vp, vp, vp, ctypes.c_float, vp, i64, vp, i64, i64, i64, ctypes.c_float, vp, i64,
                                    vp, vp, vp, vp, vp, vp]
    lib.af3k_sigmoid_gate.restype = ctypes.c_int
    lib.af3k_sigmoid_gate.argtypes = [vp, vp, vp, i64, vp]
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        lib = load()
        text = lib.af3k_strerror(code).decode()
        detail = lib.af3k_last_error_detail().decode()
        raise Af3kError(code, f"{text} ({detail})" if detail else text)


def describe_plan(desc: AttentionDesc) -> dict:
    out = (ctypes.c_int32 * 6)()
    check(load().af3k_describe_plan(ctypes.byref(desc), out))
    keys = ("rows_per_item", "kv_stages", "items", "grid", "smem_bytes", "tmem_cols")
    return dict(zip(keys, list(out)))
