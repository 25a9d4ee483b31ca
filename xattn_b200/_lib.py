"""ctypes binding of libxattn_b200.so (the C ABI in include/xattn_b200.h).

There is no CPU or eager fallback: if the library is missing or cannot be
loaded, every native call raises.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
# XATTN_B200_LIBRARY points at an alternative build of the library (development builds)
LIB_PATH = os.environ.get("XATTN_B200_LIBRARY") or os.path.join(_HERE, "libxattn_b200.so")

XATTN_DTYPE_F16, XATTN_DTYPE_BF16 = 0, 1
VIS_FULL, VIS_WINDOW, VIS_CHUNK, VIS_ALL = 0, 1, 2, 3
ABI_VERSION = 2          # XATTN_B200_ABI_VERSION of include/xattn_b200.h
BWD_PHASE_PRE, BWD_PHASE_DQ, BWD_PHASE_DKV = 1, 2, 4


class PlanArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int64), ("q_len", C.c_int64), ("k_len", C.c_int64),
        ("visibility", C.c_int), ("span", C.c_int64),
        ("strict_past", C.c_int), ("reset_positions", C.c_int),
        ("q_segment", C.c_void_p), ("k_segment", C.c_void_p),
        ("q_segment_stride", C.c_int64), ("k_segment_stride", C.c_int64),
        ("plan", C.c_void_p), ("status", C.c_void_p),
    ]


class VarlenPlanArgs(C.Structure):
    _fields_ = [
        ("total_q", C.c_int64), ("total_k", C.c_int64),
        ("num_q_seqs", C.c_int64), ("num_k_seqs", C.c_int64),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("visibility", C.c_int), ("span", C.c_int64), ("strict_past", C.c_int),
        ("plan", C.c_void_p),
    ]


class FwdArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int),
        ("batch", C.c_int64), ("q_len", C.c_int64), ("k_len", C.c_int64),
        ("q_heads", C.c_int64), ("kv_heads", C.c_int64),
        ("qk_dim", C.c_int64), ("v_dim", C.c_int64),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_strides", C.c_int64 * 3), ("k_strides", C.c_int64 * 3), ("v_strides", C.c_int64 * 3),
        ("scale", C.c_float), ("high_precision", C.c_int),
        ("plan", C.c_void_p),
        ("y", C.c_void_p), ("lse", C.c_void_p), ("y_state", C.c_void_p),
        ("status", C.c_void_p), ("anchor", C.c_void_p),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int),
        ("batch", C.c_int64), ("q_len", C.c_int64), ("k_len", C.c_int64),
        ("q_heads", C.c_int64), ("kv_heads", C.c_int64),
        ("qk_dim", C.c_int64), ("v_dim", C.c_int64),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("y", C.c_void_p), ("dy", C.c_void_p),
        ("q_strides", C.c_int64 * 3), ("k_strides", C.c_int64 * 3), ("v_strides", C.c_int64 * 3),
        ("y_strides", C.c_int64 * 3), ("dy_strides", C.c_int64 * 3),
        ("lse", C.c_void_p), ("scale", C.c_float),
        ("plan", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("workspace", C.c_void_p), ("status", C.c_void_p),
        ("high_precision", C.c_int), ("anchor", C.c_void_p), ("grad_unscale", C.c_void_p),
        ("phases", C.c_int),
    ]


class GateArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("neg_is_f32", C.c_int),
        ("rows", C.c_int64), ("q_heads", C.c_int64), ("kv_heads", C.c_int64), ("v_dim", C.c_int64),
        ("g", C.c_void_p), ("neg_read", C.c_void_p), ("read", C.c_void_p), ("y", C.c_void_p),
        ("dy", C.c_void_p), ("dneg_read", C.c_void_p), ("dg", C.c_void_p),
        ("value_groups", C.c_int64),
    ]


class ConstantKeyArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int),
        ("batch", C.c_int64), ("q_len", C.c_int64), ("k_len", C.c_int64),
        ("q_heads", C.c_int64), ("kv_heads", C.c_int64), ("qk_dim", C.c_int64),
        ("dq", C.c_void_p), ("k", C.c_void_p), ("k_strides", C.c_int64 * 3),
        ("plan", C.c_void_p), ("workspace", C.c_void_p),
    ]


class MergeArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int),
        ("batch", C.c_int64), ("k_len", C.c_int64), ("kv_heads", C.c_int64), ("dim", C.c_int64),
        ("a", C.c_void_p), ("b", C.c_void_p), ("tail", C.c_void_p), ("tail_len", C.c_int64),
        ("out", C.c_void_p),
    ]


class MergeOutputsArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int64), ("rows", C.c_int64), ("heads", C.c_int64), ("v_dim", C.c_int64),
        ("acc_rows", C.c_int64), ("row_offset", C.c_int64),
        ("y_acc", C.c_void_p), ("lse_acc", C.c_void_p), ("y_part", C.c_void_p), ("lse_part", C.c_void_p),
    ]


_lock = threading.Lock()
_lib: Optional[C.CDLL] = None

# name -> (restype, argtypes); every symbol include/xattn_b200.h declares
SYMBOLS = {
    "xattn_b200_abi_version": (C.c_int, []),
    "xattn_b200_last_error": (C.c_char_p, []),
    "xattn_b200_plan_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "xattn_b200_build_plan": (C.c_int, [C.POINTER(PlanArgs), C.c_void_p]),
    "xattn_b200_build_varlen_plan": (C.c_int, [C.POINTER(VarlenPlanArgs), C.c_void_p]),
    "xattn_b200_fwd": (C.c_int, [C.POINTER(FwdArgs), C.c_void_p]),
    "xattn_b200_fwd_split_suggest": (C.c_int64, [C.c_int64] * 6),
    "xattn_b200_fwd_split_workspace_bytes": (C.c_size_t, [C.c_int64] * 5),
    "xattn_b200_fwd_split": (C.c_int, [C.POINTER(FwdArgs), C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p]),
    "xattn_b200_bwd_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "xattn_b200_bwd_workspace_bytes_hp": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "xattn_b200_bwd": (C.c_int, [C.POINTER(BwdArgs), C.c_void_p]),
    "xattn_b200_bwd_static_scratch": (C.c_int, [C.POINTER(BwdArgs), C.c_void_p]),
    "xattn_b200_softdelta_gate_fwd": (C.c_int, [C.POINTER(GateArgs), C.c_void_p]),
    "xattn_b200_softdelta_gate_bwd": (C.c_int, [C.POINTER(GateArgs), C.c_void_p]),
    "xattn_b200_zero_constant_key_rows": (C.c_int, [C.POINTER(ConstantKeyArgs), C.c_void_p]),
    "xattn_b200_softdelta_merge_gradients": (C.c_int, [C.POINTER(MergeArgs), C.c_void_p]),
    "xattn_b200_profile_enable": (C.c_int, [C.c_int]),
    "xattn_b200_profile_read": (C.c_int, [C.POINTER(C.c_int), C.POINTER(C.c_float), C.c_int]),
    "xattn_b200_merge_partial_outputs": (C.c_int, [C.POINTER(MergeOutputsArgs), C.c_void_p]),
    "xattn_b200_selftest_wait_timeout": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p]),
    "xattn_b200_check_status": (C.c_int, [C.c_void_p, C.c_void_p]),
}


def load() -> C.CDLL:
    """Load the shared library once; raise ImportError with build instructions when absent."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing. Build it with `python -m xattn_b200.build` "
                "(needs nvcc; sm_100a only). There is no CPU fallback."
            )
        lib = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.xattn_b200_abi_version() != ABI_VERSION:
            raise ImportError("libxattn_b200.so has an unexpected ABI version; rebuild it")
        _lib = lib
        return lib


def last_error() -> str:
    msg = load().xattn_b200_last_error()
    return msg.decode() if msg else ""


def check(code: int, what: str) -> None:
    """Turn a negative return code into the exception the reference's TORCH_CHECK would raise."""
    if code == 0:
        return
    raise RuntimeError(f"{what}: {last_error()} (code {code})")
