"""ctypes binding of libfba_b200.so (declared in include/fba.h).

This module is the only place that touches the C ABI.  It stands where the reference's
``from flex_block_attn_cuda import attn_forward, attn_backward`` stood
(reference flex_block_attn/flex_block_attn_interface.py:4).  There is no CPU fallback: if the
library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB = None
FBA_ERR_TIMEOUT = -4
FBA_ERR_TOO_LARGE = -5
LIB_PATH = Path(__file__).resolve().parent / "libfba_b200.so"

EXPORTED_SYMBOLS = (
    "fba_abi_version",
    "fba_last_error",
    "fba_launch_count",
    "fba_set_timing_events",
    "fba_check_status",
    "fba_selftest_wait_timeout",
    "fba_fwd_order",
    "fba_bwd_order",
    "fba_attn_workspace_bytes",
    "fba_attn_forward",
    "fba_attn_backward",
    "fba_build_index",
    "fba_build_tile_lists",
    "fba_sta_index",
    "fba_ssta_scratch_floats",
    "fba_ssta_index",
    "fba_tile_major",
    "fba_fwd",
    "fba_fwd_scaled",
    "fba_quantize_kv_e4m3",
    "fba_fwd_fp8kv",
    "fba_bwd_scratch_bytes",
    "fba_bwd",
    "fba_bwd_scaled",
    "fba_bwd_ex",
    "fba_set_bwd_kernel",
    "fba_bwd_static_scratch_max_rows",
    "fba_bwd_static_scratch",
    "fba_peer_alloc",
    "fba_peer_free",
    "fba_peer_export",
    "fba_peer_open",
    "fba_peer_close",
    "fba_peer_exchange",
)


class FbaList(ctypes.Structure):
    """Mirror of ``fba_list_t``."""

    _fields_ = [
        ("idx", ctypes.c_void_p),
        ("cnt", ctypes.c_void_p),
        ("msk", ctypes.c_void_p),
        ("stride", ctypes.c_int32),
        ("rows_per_bh", ctypes.c_int32),
        ("bh_stride", ctypes.c_int32),
        ("rows_div", ctypes.c_int32),
        ("sub", ctypes.c_int32),
        ("order", ctypes.c_void_p),
    ]

    def __init__(self, idx=None, cnt=None, msk=None, stride=0, rows_per_bh=0, bh_stride=0, rows_div=1, sub=1,
                 order=None):
        super().__init__(idx, cnt, msk, stride, rows_per_bh, bh_stride, rows_div, sub, order)


def lib() -> ctypes.CDLL:
    """Load the shared library once (building it first when FBA_AUTO_BUILD=1 and it is missing)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not LIB_PATH.exists() and os.environ.get("FBA_AUTO_BUILD", "0") == "1":
        from .build import build_library

        build_library()
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flex_block_attn_b200.build` "
            "(there is no CPU or PyTorch fallback for this operator)"
        )
    L = ctypes.CDLL(str(LIB_PATH))
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    L.fba_abi_version.restype = i32
    L.fba_abi_version.argtypes = []
    L.fba_last_error.restype = ctypes.c_char_p
    L.fba_last_error.argtypes = []
    L.fba_launch_count.restype = ctypes.c_uint64
    L.fba_launch_count.argtypes = []
    L.fba_set_timing_events.restype = i32
    L.fba_set_timing_events.argtypes = [i32, vp, vp]
    L.fba_check_status.restype = i32
    L.fba_check_status.argtypes = [vp, vp]
    L.fba_selftest_wait_timeout.restype = i32
    L.fba_selftest_wait_timeout.argtypes = [vp, ctypes.c_int64, vp, vp]
    L.fba_fwd_order.restype = i32
    L.fba_fwd_order.argtypes = [ctypes.POINTER(FbaList), i32, i32, i32, vp, vp]
    L.fba_bwd_order.restype = i32
    L.fba_bwd_order.argtypes = [ctypes.POINTER(FbaList), i32, i32, i32, i32, vp, vp]
    L.fba_attn_workspace_bytes.restype = i32
    L.fba_attn_workspace_bytes.argtypes = [i32] * 9 + [ctypes.POINTER(ctypes.c_uint64)]
    L.fba_attn_forward.restype = i32
    L.fba_attn_forward.argtypes = [vp] * 5 + [i32] * 7 + [vp, vp, i32, i32, vp, ctypes.c_uint64, vp, vp]
    L.fba_attn_backward.restype = i32
    L.fba_attn_backward.argtypes = [vp] * 9 + [i32] * 7 + [vp, vp, i32, i32, vp, ctypes.c_uint64, vp, vp]
    L.fba_build_index.restype = i32
    L.fba_build_index.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp]
    L.fba_build_tile_lists.restype = i32
    L.fba_build_tile_lists.argtypes = [vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp]
    L.fba_sta_index.restype = i32
    L.fba_sta_index.argtypes = [i32] * 6 + [vp, vp, vp]
    L.fba_ssta_scratch_floats.restype = i32
    L.fba_ssta_scratch_floats.argtypes = [i32] * 5 + [ctypes.POINTER(ctypes.c_uint64)]
    L.fba_ssta_index.restype = i32
    L.fba_ssta_index.argtypes = [vp, vp] + [i32] * 14 + [vp] * 7
    L.fba_tile_major.restype = i32
    L.fba_tile_major.argtypes = [vp, vp] + [i32] * 9 + [vp]
    L.fba_fwd.restype = i32
    L.fba_fwd.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, ctypes.POINTER(FbaList), vp, vp]
    L.fba_fwd_scaled.restype = i32
    L.fba_fwd_scaled.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, ctypes.POINTER(FbaList),
                                 ctypes.c_float, vp, vp]
    L.fba_quantize_kv_e4m3.restype = i32
    L.fba_quantize_kv_e4m3.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
    L.fba_fwd_fp8kv.restype = i32
    L.fba_fwd_fp8kv.argtypes = [vp] * 5 + [i32, vp, vp] + [i32] * 5 + [ctypes.POINTER(FbaList), ctypes.c_float, vp, vp]
    L.fba_bwd_scratch_bytes.restype = i32
    L.fba_bwd_scratch_bytes.argtypes = [i32, i32, i32, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
    L.fba_bwd.restype = i32
    L.fba_bwd.argtypes = [vp] * 9 + [i32] * 5 + [ctypes.POINTER(FbaList), vp, vp, vp, vp]
    L.fba_bwd_scaled.restype = i32
    L.fba_bwd_scaled.argtypes = [vp] * 9 + [i32] * 5 + [ctypes.POINTER(FbaList), ctypes.c_float, vp, vp, vp, vp]
    L.fba_bwd_ex.restype = i32
    L.fba_bwd_ex.argtypes = [vp] * 9 + [i32] * 5 + [ctypes.POINTER(FbaList), ctypes.POINTER(FbaList), ctypes.c_float, i32,
                                                     vp, vp, vp, vp]
    L.fba_set_bwd_kernel.restype = i32
    L.fba_set_bwd_kernel.argtypes = [i32]
    L.fba_bwd_static_scratch_max_rows.restype = ctypes.c_uint64
    L.fba_bwd_static_scratch_max_rows.argtypes = []
    L.fba_bwd_static_scratch.restype = i32
    L.fba_bwd_static_scratch.argtypes = [vp] * 9 + [i32] * 5 + [ctypes.POINTER(FbaList), vp, vp]
    L.fba_peer_alloc.restype = i32
    L.fba_peer_alloc.argtypes = [ctypes.c_uint64, ctypes.POINTER(vp)]
    L.fba_peer_free.restype = i32
    L.fba_peer_free.argtypes = [vp]
    L.fba_peer_export.restype = i32
    L.fba_peer_export.argtypes = [vp, ctypes.c_char_p]
    L.fba_peer_open.restype = i32
    L.fba_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.fba_peer_close.restype = i32
    L.fba_peer_close.argtypes = [vp]
    L.fba_peer_exchange.restype = i32
    L.fba_peer_exchange.argtypes = [vp, ctypes.POINTER(vp)] + [i32] * 11 + [vp]
    if L.fba_abi_version() != 2:
        raise RuntimeError("libfba_b200.so has an unexpected ABI version")
    _LIB = L
    return L


def check(rc: int, what: str) -> None:
    """Turn a non-zero status code into a RuntimeError carrying the library's message."""
    if rc != 0:
        msg = lib().fba_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed with status {rc}: {msg}")
