"""Sliding-window attention (FlashSWA): public ops with the reference's signatures
(xattn/ops/sliding_window_attention.py:31-185) plus the packed-varlen helpers its tests use
(xattn/ops/_causal_attention.py:1032-1188)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _native
from . import _core
from ._validation import (dispatch_nonpositive_scale, resolve_scale, validate_attention_scale,
                          validate_dimensions, validate_high_precision_level, validate_window_size)
from ._varlen import VarlenFunction, validate_packed

__all__ = ["flash_swa", "flash_swa_bwd", "flash_swa_fwd"]


def flash_swa(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    window_size: int,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    *,
    segment_idx: Optional[Tensor] = None,
    bos_mask: Optional[Tensor] = None,
    backend: str = "auto",
    deterministic: bool = False,
    high_precision_level: int = 0,
) -> Tensor:
    """Causal sliding-window attention with autograd.

    ``window_size`` is an inclusive left radius: query ``i`` sees keys in
    ``[i + Lk - Lq - window_size, i + Lk - Lq]`` of the total K/V (``prev_k`` / ``prev_v``, any
    positive length, come first).  Segment equality is applied after alignment; ``segment_idx``
    and ``bos_mask`` describe the total K/V and Q uses their suffix.
    """
    validate_high_precision_level(high_precision_level, api_name="flash_swa")
    validate_attention_scale(scale)
    validate_dimensions(q, v, backend, api_name="flash_swa")
    if scale is not None and float(scale) <= 0:
        return dispatch_nonpositive_scale(flash_swa, locals())
    validate_window_size(window_size)
    return _core.attention(
        q, k, v, _core.Support("window", window_size), scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
        segment_idx=segment_idx, bos_mask=bos_mask, backend=backend, deterministic=deterministic,
        high_precision_level=high_precision_level, api_name="flash_swa",
    )


def flash_swa_fwd(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    window_size: int,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    *,
    segment_idx: Optional[Tensor] = None,
    bos_mask: Optional[Tensor] = None,
    backend: str = "auto",
    high_precision_level: int = 0,
) -> Tuple[Tensor, Tensor]:
    """``(y, lse)``: ``y`` in the input dtype, ``lse`` FP32 ``[B, Hq, Lq]``."""
    validate_high_precision_level(high_precision_level, api_name="flash_swa_fwd")
    validate_attention_scale(scale)
    validate_dimensions(q, v, backend, api_name="flash_swa_fwd")
    if scale is not None and float(scale) <= 0:
        return dispatch_nonpositive_scale(flash_swa_fwd, locals())
    validate_window_size(window_size)
    return _core.attention_fwd(
        q, k, v, _core.Support("window", window_size), scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
        segment_idx=segment_idx, bos_mask=bos_mask, backend=backend,
        high_precision_level=high_precision_level, api_name="flash_swa_fwd",
    )


def flash_swa_bwd(
    y_grad: Tensor,
    q: Tensor,
    k: Tensor,
    v: Tensor,
    y: Tensor,
    lse: Tensor,
    window_size: int,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    *,
    segment_idx: Optional[Tensor] = None,
    bos_mask: Optional[Tensor] = None,
    backend: str = "auto",
    deterministic: bool = False,
    high_precision_level: int = 0,
) -> Tuple[Tensor, Tensor, Tensor, Optional[Tensor], Optional[Tensor]]:
    """``(dq, dk, dv, dprev_k, dprev_v)``; the last two are None without previous K/V."""
    validate_high_precision_level(high_precision_level, api_name="flash_swa_bwd")
    validate_attention_scale(scale)
    validate_dimensions(q, v, backend, api_name="flash_swa_bwd")
    if scale is not None and float(scale) <= 0:
        return dispatch_nonpositive_scale(flash_swa_bwd, locals())
    validate_window_size(window_size)
    return _core.attention_bwd(
        y_grad, q, k, v, y, lse, _core.Support("window", window_size), scale, prev_k, prev_v,
        q_segment_idx, k_segment_idx, segment_idx=segment_idx, bos_mask=bos_mask, backend=backend,
        deterministic=deterministic, high_precision_level=high_precision_level, api_name="flash_swa_bwd",
    )


# ---- packed varlen (internal in the reference too) -------------------------------------------

def _support(window_size: Optional[int]) -> _core.Support:
    return _core.Support("full") if window_size is None else _core.Support("window", window_size)


def _flash_swa_varlen(q, k, v, window_size, scale=None, *, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                      max_seqlen_k, backend="auto", deterministic=False) -> Tensor:
    """Packed ``[T, H, D]`` inputs; Q sequence ``r`` is right-aligned to its K sequence and no
    attention crosses a cu_seqlens boundary."""
    validate_packed(q, k, v, window_size, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                    api_name="_flash_swa_varlen", span_name="window_size")
    return VarlenFunction.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, _support(window_size), resolve_scale(q, scale))


def _flash_swa_varlen_fwd(q, k, v, window_size, scale=None, *, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                          max_seqlen_k, backend="auto", output_state=None) -> Tuple[Tensor, Tensor]:
    validate_packed(q, k, v, window_size, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                    api_name="_flash_swa_varlen_fwd", span_name="window_size")
    from ._varlen import varlen_forward
    with torch.no_grad():
        return varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, _support(window_size), resolve_scale(q, scale),
                              output_state=output_state)


def _flash_swa_varlen_bwd(y_grad, q, k, v, y, lse, window_size, scale=None, *, cu_seqlens_q, cu_seqlens_k,
                          max_seqlen_q, max_seqlen_k, backend="auto", deterministic=False):
    validate_packed(q, k, v, window_size, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                    api_name="_flash_swa_varlen_bwd", span_name="window_size")
    from ._varlen import varlen_backward
    with torch.no_grad():
        return varlen_backward(y_grad, q, k, v, y, lse, cu_seqlens_q, cu_seqlens_k, _support(window_size),
                               resolve_scale(q, scale))
