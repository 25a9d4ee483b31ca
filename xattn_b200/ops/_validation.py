"""Argument validation shared by every public op.

Mirrors the reference's checks that run before any tensor is touched
(xattn/ops/_backward_precision.py:5-56, xattn/ops/_attention_core.py:208-229,
xattn/ops/_causal_attention.py:111-198, xattn/ops/_segment_metadata.py:7-75,
xattn/ops/_bos_metadata.py:7-22): same exception types, same message keywords
(``high_precision_level``, ``multiples of 8``, ``scale must be finite``,
``Q/K/V dtype``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor

# The reference's callers pass backend="sm90"; this build has exactly one
# backend, so every accepted spelling selects the sm_100a kernels.
_BACKENDS = ("", "auto", "sm90", "sm100", "sm100a")


def normalize_backend(backend: str, api_name: str) -> str:
    if not isinstance(backend, str):
        raise TypeError(f"{api_name} backend must be a string")
    name = backend.strip().lower()
    if name not in _BACKENDS:
        raise ValueError(f"{api_name} backend must be one of: auto, sm90, sm100 (got {backend!r})")
    return name


def validate_high_precision_level(level, *, api_name: str = "attention") -> int:
    """0, or 1 for the high-precision softmax and backward.  ``bool`` is not an integer here."""
    if isinstance(level, bool) or not isinstance(level, int):
        raise TypeError(f"{api_name} high_precision_level must be 0 or 1")
    if level not in (0, 1):
        raise ValueError(f"{api_name} high_precision_level must be 0 or 1, got {level}")
    return level


def validate_attention_scale(scale) -> None:
    if scale is not None and not math.isfinite(float(scale)):
        raise ValueError("attention scale must be finite")


def validate_dimensions(q, v, backend, *, api_name: str) -> None:
    """Reject head dimensions TMA cannot describe, before any descriptor is built."""
    if not isinstance(q, Tensor) or not isinstance(v, Tensor):
        return  # rank / type diagnostics belong to the input validator
    if not q.is_cuda or q.dim() != 4 or v.dim() != 4:
        return
    dim, width = q.shape[-1], v.shape[-1]
    if q.shape[0] <= 0:
        raise ValueError(f"{api_name} batch size must be positive")
    if not (0 < dim <= 256 and 0 < width <= 256 and dim % 8 == 0 and width % 8 == 0):
        raise ValueError(
            f"{api_name} requires Q/K and V head dimensions to be multiples of 8 in [8, 256]; "
            f"got D={dim}, V={width}"
        )


def validate_attention_output(y: Tensor, q: Tensor) -> None:
    if y.dtype != q.dtype:
        raise ValueError(f"attention output y must have the Q/K/V dtype {q.dtype}, got {y.dtype}")


def validate_saved_state(y: Tensor, lse: Tensor, q: Tensor, v: Tensor) -> None:
    if q.dim() != 4 or v.dim() != 4:
        raise ValueError("attention Q/V must be rank-four tensors")
    if y.shape != (*q.shape[:-1], v.shape[-1]) or y.device != q.device:
        raise ValueError("saved attention output has incompatible shape or device")
    if lse.shape != (q.shape[0], q.shape[2], q.shape[1]) or lse.device != q.device or lse.dtype != torch.float32:
        raise ValueError("attention LSE must be FP32 [B,Hq,Nq] on Q's device")


def resolve_scale(q: Tensor, scale: Optional[float]) -> float:
    return 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)


def validate_window_size(window_size, api_name: str = "flash_swa") -> None:
    if isinstance(window_size, bool) or not isinstance(window_size, int):
        raise TypeError(f"{api_name} window_size must be an integer")
    if window_size < 0:
        raise ValueError(f"{api_name} window_size must be nonnegative")


def validate_chunk_size(chunk_size, api_name: str = "flash_sca") -> None:
    if isinstance(chunk_size, bool) or not isinstance(chunk_size, int):
        raise TypeError(f"{api_name} chunk_size must be an integer")
    if chunk_size <= 0:
        raise ValueError(f"{api_name} chunk_size must be positive")


def validate_qkv(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    prev_k: Optional[Tensor],
    prev_v: Optional[Tensor],
    *,
    api_name: str,
) -> int:
    """Shape / dtype / device contract of the dense layouts; returns the previous-K/V length."""
    for t in (q, k, v):
        if not isinstance(t, Tensor):
            raise TypeError(f"{api_name} q/k/v must be tensors")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError(f"{api_name} expects 4D q/k/v tensors laid out [B, L, H, D]")
    if q.device != k.device or q.device != v.device:
        raise ValueError(f"{api_name} q/k/v must share a device")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError(f"{api_name} q/k/v must share a dtype")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"{api_name} supports only fp16 and bf16 inputs")
    if q.shape[0] != k.shape[0] or k.shape[:2] != v.shape[:2]:
        raise ValueError(f"{api_name} batch dimensions and k/v lengths must match")
    if not 0 < q.shape[1] <= k.shape[1]:
        raise ValueError(f"{api_name} requires 0 < q length <= k/v length")
    if k.shape[2] != v.shape[2]:
        raise ValueError(f"{api_name} k/v head counts must match")
    if q.shape[2] <= 0 or k.shape[2] <= 0:
        raise ValueError(f"{api_name} q and KV head counts must be positive")
    if q.shape[2] % k.shape[2] != 0:
        raise ValueError(f"{api_name} q head count must be divisible by the KV head count")
    if q.shape[-1] != k.shape[-1] or q.shape[-1] <= 0:
        raise ValueError(f"{api_name} q/k head dims must match and be positive")
    if v.shape[-1] <= 0:
        raise ValueError(f"{api_name} value head dim must be positive")
    if (prev_k is None) != (prev_v is None):
        raise ValueError(f"{api_name} prev_k and prev_v must be provided together")
    if prev_k is None:
        return 0
    if prev_k.dim() != 4 or prev_v.dim() != 4:
        raise ValueError(f"{api_name} prev_k/prev_v must be 4D tensors")
    if prev_k.device != q.device or prev_v.device != q.device:
        raise ValueError(f"{api_name} previous and current K/V must share a device")
    if prev_k.dtype != q.dtype or prev_v.dtype != q.dtype:
        raise ValueError(f"{api_name} previous and current K/V must share a dtype")
    if (
        prev_k.shape[0] != q.shape[0]
        or prev_v.shape[0] != q.shape[0]
        or prev_k.shape[1] != prev_v.shape[1]
        or prev_k.shape[1] <= 0
        or prev_k.shape[2:] != k.shape[2:]
        or prev_v.shape[2:] != v.shape[2:]
    ):
        raise ValueError(f"{api_name} previous K/V shapes are incompatible with Q/K/V")
    return prev_k.shape[1]


def validate_gate_and_reader(q: Tensor, k: Tensor, g, k_read, deterministic, *, api_name: str) -> None:
    """What SoftDelta adds to the q/k/v contract: one gate logit per (token, query head), an optional
    second reader shaped like the aligned keys, both in q's dtype on q's device
    (xattn/ops/softdelta_attention.py:101-166; message keywords ``g must have shape`` and
    ``k_read must have shape`` are pinned by the reference's tests)."""
    if not isinstance(deterministic, bool):
        raise TypeError(f"{api_name} deterministic must be a bool")
    extras = {"g": (g, tuple(q.shape[:3])), "k_read": (k_read, (q.shape[0], q.shape[1], k.shape[2], q.shape[3]))}
    for name, (tensor, shape) in extras.items():
        if tensor is None and name == "k_read":
            continue
        if not isinstance(tensor, Tensor):
            raise TypeError(f"{api_name} {name} must be a tensor")
        if tensor.device != q.device:
            raise ValueError(f"{api_name} q/k/v/g/k_read must share a device")
        if tensor.dtype != q.dtype:
            raise ValueError(f"{api_name} q/k/v/g/k_read must share a dtype")
        if tuple(tensor.shape) != shape:
            raise ValueError(f"{api_name} {name} must have shape {list(shape)}")


def resolve_segments(
    q: Tensor,
    k_length: int,
    segment_idx: Optional[Tensor],
    q_segment_idx: Optional[Tensor],
    k_segment_idx: Optional[Tensor],
    bos_mask: Optional[Tensor],
    *,
    api_name: str,
) -> Tuple[Optional[Tensor], Optional[Tensor]]:
    """The three exclusive metadata forms -> (q ids [B, Lq], k ids [B, k_length]) or (None, None).

    ``segment_idx`` labels all keys and its suffix labels Q; a BOS mask becomes ids by a running
    count of its set bits (xattn/ops/_bos_metadata.py:84-90); explicit Q / K ids pass through.
    No device value is read.

    Contract: the key ids of a row must never decrease (the keys carrying one id are one contiguous run,
    which the plan kernels locate by binary search; the reference's kernels assume the same,
    csrc/attention/partition/segment_index.h:362-363).  BOS masks satisfy it by construction.  The plan
    kernels compare neighbouring key ids on the device and a violation surfaces as a ``RuntimeError``
    naming the batch row, at the call itself with ``XATTN_B200_SYNC_CHECK=1``, else at the next call or
    ``check_status()``.
    """
    batch, q_length = q.shape[0], q.shape[1]
    if bos_mask is not None:
        if segment_idx is not None or q_segment_idx is not None or k_segment_idx is not None:
            raise ValueError("BOS masks and segment indices are mutually exclusive")
        if (
            not isinstance(bos_mask, Tensor)
            or bos_mask.device != q.device
            or bos_mask.dtype != torch.bool
            or tuple(bos_mask.shape) != (batch, k_length)
        ):
            raise ValueError(
                f"bos_mask must be a bool tensor on the Q/K/V device with shape {[batch, k_length]}"
            )
        k_ids = bos_mask.cumsum(dim=1, dtype=torch.int64)
        return k_ids[:, k_length - q_length:], k_ids
    if segment_idx is not None:
        if q_segment_idx is not None or k_segment_idx is not None:
            raise ValueError("segment_idx cannot be combined with q_segment_idx or k_segment_idx")
        if tuple(segment_idx.shape) != (batch, k_length):
            raise ValueError(f"segment_idx must have shape [{batch}, {k_length}]")
        q_segment_idx = segment_idx if q_length == k_length else segment_idx[:, -q_length:]
        k_segment_idx = segment_idx
    if (q_segment_idx is None) != (k_segment_idx is None):
        raise ValueError("q_segment_idx and k_segment_idx must be provided together")
    if q_segment_idx is None:
        return None, None
    if q_segment_idx.dtype != torch.int64:
        raise ValueError(f"{api_name} q_segment_idx must be torch.int64")
    if k_segment_idx.dtype != torch.int64:
        raise ValueError(f"{api_name} k_segment_idx must be torch.int64")
    if q_segment_idx.device != q.device or k_segment_idx.device != q.device:
        raise ValueError(f"{api_name} segment metadata must share the Q/K/V device")
    if tuple(q_segment_idx.shape) != (batch, q_length):
        raise ValueError(f"{api_name} q_segment_idx must have shape [{batch}, {q_length}]")
    if tuple(k_segment_idx.shape) != (batch, k_length):
        raise ValueError(f"{api_name} k_segment_idx must have shape [{batch}, {k_length}]")
    return q_segment_idx, k_segment_idx


def dispatch_nonpositive_scale(function, arguments):
    """Finite scale <= 0 runs as a positive scale on -q (or 0*q); exact for fp16 / bf16 inputs
    (xattn/ops/_backward_precision.py:40-56).  Autograd sees the Q transform; a standalone
    backward gets the chain-rule sign applied to dq here."""
    options = dict(arguments)
    scale = float(options["scale"])
    q = options["q"]
    options["q"] = -q if scale < 0 else q * 0
    options["scale"] = -scale if scale < 0 else 1.0
    result = function(**options)
    if function.__name__.endswith("_bwd"):
        dq = -result[0] if scale < 0 else torch.zeros_like(result[0])
        result = (dq, *result[1:])
    return result
