"""Sliding-chunk attention (FlashSCA): public ops with the reference's signatures
(xattn/ops/sliding_chunk_attention.py:2300-2662).

Query at position ``p`` sees the keys of its own chunk up to ``p`` and the whole chunk before it:
``[(p // c - 1) * c, p]``.  Positions are global (previous K/V first) or, with
``reset_chunk_pos_per_seq``, restart in every segment run.  The reference needs separate
metadata kernels, a BOS plan with a host synchronisation, a row-aligned varlen route and a
"matched reset" pack/scatter path for independent Q / K ids
(csrc/flash_sca/hopper/sliding_chunk_attention.cu:1942-2064,2194-2642,
xattn/ops/_sca_segment_alignment.py:54-182); here all of them are one mask plan.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _core
from ._validation import (dispatch_nonpositive_scale, resolve_scale, validate_attention_scale,
                          validate_chunk_size, validate_dimensions, validate_high_precision_level)
from ._varlen import VarlenFunction, validate_packed, varlen_backward, varlen_forward

__all__ = ["flash_sca", "flash_sca_bwd", "flash_sca_fwd", "flash_sca_sm90_available"]


def _resolve_attn_method(attn_method: str) -> str:
    if not isinstance(attn_method, str):
        raise TypeError("attn_method must be a string")
    method = attn_method.strip().lower().replace("-", "_")
    if method not in ("default", "sda"):
        raise ValueError("attn_method must be one of: default, sda")
    if method == "sda":
        raise NotImplementedError(
            "attn_method='sda' is reserved for SoftDelta attention output; "
            "use sliding_chunk_softdelta_attention(q, k, v, g, ...)"
        )
    return method


def _support(chunk_size, reset, prev_k, api_name) -> _core.Support:
    validate_chunk_size(chunk_size, api_name)
    if not isinstance(reset, bool):
        raise TypeError(f"{api_name} reset_chunk_pos_per_seq must be a bool")
    if prev_k is not None and isinstance(prev_k, Tensor) and prev_k.dim() == 4 and prev_k.shape[1] != chunk_size:
        raise ValueError(f"{api_name} prev_k/prev_v sequence length must equal chunk_size")
    return _core.Support("chunk", chunk_size, reset)


def flash_sca(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    chunk_size: int,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    *,
    segment_idx: Optional[Tensor] = None,
    bos_mask: Optional[Tensor] = None,
    backend: str = "auto",
    reset_chunk_pos_per_seq: bool = False,
    deterministic: bool = False,
    attn_method: str = "default",
    high_precision_level: int = 0,
) -> Tensor:
    """Sliding-chunk attention with dense, segment-id or BOS metadata, with autograd.

    Q may be shorter than the current K/V and is aligned to the end of the total K/V (previous K/V,
    exactly ``chunk_size`` tokens when given, comes first).  With reset positions, matching
    segment ids align at their segment ends instead.
    """
    validate_high_precision_level(high_precision_level, api_name="flash_sca")
    validate_attention_scale(scale)
    validate_dimensions(q, v, backend, api_name="flash_sca")
    if scale is not None and float(scale) <= 0:
        return dispatch_nonpositive_scale(flash_sca, locals())
    _resolve_attn_method(attn_method)
    support = _support(chunk_size, reset_chunk_pos_per_seq, prev_k, "flash_sca")
    return _core.attention(
        q, k, v, support, scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
        segment_idx=segment_idx, bos_mask=bos_mask, backend=backend, deterministic=deterministic,
        high_precision_level=high_precision_level, api_name="flash_sca",
    )


def flash_sca_fwd(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    chunk_size: int,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    *,
    segment_idx: Optional[Tensor] = None,
    bos_mask: Optional[Tensor] = None,
    backend: str = "auto",
    reset_chunk_pos_per_seq: bool = False,
    attn_method: str = "default",
    high_precision_level: int = 0,
) -> Tuple[Tensor, Tensor]:
    """``(y, lse)``: ``y`` in the input dtype, ``lse`` FP32 ``[B, Hq, Lq]``."""
    validate_high_precision_level(high_precision_level, api_name="flash_sca_fwd")
    validate_attention_scale(scale)
    validate_dimensions(q, v, backend, api_name="flash_sca_fwd")
    if scale is not None and float(scale) <= 0:
        return dispatch_nonpositive_scale(flash_sca_fwd, locals())
    _resolve_attn_method(attn_method)
    support = _support(chunk_size, reset_chunk_pos_per_seq, prev_k, "flash_sca_fwd")
    return _core.attention_fwd(
        q, k, v, support, scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
        segment_idx=segment_idx, bos_mask=bos_mask, backend=backend,
        high_precision_level=high_precision_level, api_name="flash_sca_fwd",
    )


def flash_sca_bwd(
    y_grad: Tensor,
    q: Tensor,
    k: Tensor,
    v: Tensor,
    y: Tensor,
    lse: Tensor,
    chunk_size: int,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    *,
    segment_idx: Optional[Tensor] = None,
    bos_mask: Optional[Tensor] = None,
    backend: str = "auto",
    reset_chunk_pos_per_seq: bool = False,
    deterministic: bool = False,
    attn_method: str = "default",
    high_precision_level: int = 0,
) -> Tuple[Tensor, Tensor, Tensor, Optional[Tensor], Optional[Tensor]]:
    """``(dq, dk, dv, dprev_k, dprev_v)``; the last two are None without previous K/V."""
    validate_high_precision_level(high_precision_level, api_name="flash_sca_bwd")
    validate_attention_scale(scale)
    validate_dimensions(q, v, backend, api_name="flash_sca_bwd")
    if scale is not None and float(scale) <= 0:
        return dispatch_nonpositive_scale(flash_sca_bwd, locals())
    _resolve_attn_method(attn_method)
    support = _support(chunk_size, reset_chunk_pos_per_seq, prev_k, "flash_sca_bwd")
    return _core.attention_bwd(
        y_grad, q, k, v, y, lse, support, scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
        segment_idx=segment_idx, bos_mask=bos_mask, backend=backend, deterministic=deterministic,
        high_precision_level=high_precision_level, api_name="flash_sca_bwd",
    )


def flash_sca_sm90_available(q: Tensor) -> bool:
    """Whether the fused kernels can run on ``q``'s device.  The name is the reference's
    (xattn/ops/sliding_chunk_attention.py:2661); in this build it means an sm_100 GPU with the
    library loaded."""
    if not isinstance(q, Tensor) or not q.is_cuda:
        return False
    from .. import _lib
    try:
        _lib.load()
    except ImportError:
        return False
    return torch.cuda.get_device_capability(q.device)[0] == 10


# ---- packed varlen (internal in the reference too, xattn/ops/sliding_chunk_attention.py:1122-1175) ----

def _varlen_support(chunk_size, reset, position_offsets, api_name) -> _core.Support:
    if position_offsets is not None or not reset:
        raise NotImplementedError(
            f"{api_name}: packed inputs restart chunk positions in every sequence in this build "
            "(pass reset_chunk_pos_per_seq=True and no position_offsets)"
        )
    return _core.Support("chunk", chunk_size, True)


def _flash_sca_varlen(q, k, v, chunk_size, scale=None, *, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                      max_seqlen_k, position_offsets=None, backend="auto", reset_chunk_pos_per_seq=False,
                      deterministic=False, attn_method="default") -> Tensor:
    _resolve_attn_method(attn_method)
    validate_packed(q, k, v, chunk_size, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                    api_name="_flash_sca_varlen", span_name="chunk_size")
    support = _varlen_support(chunk_size, reset_chunk_pos_per_seq, position_offsets, "_flash_sca_varlen")
    return VarlenFunction.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, support, resolve_scale(q, scale))


def _flash_sca_varlen_fwd(q, k, v, chunk_size, scale=None, *, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                          max_seqlen_k, position_offsets=None, backend="auto", reset_chunk_pos_per_seq=False,
                          attn_method="default"):
    _resolve_attn_method(attn_method)
    validate_packed(q, k, v, chunk_size, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                    api_name="_flash_sca_varlen_fwd", span_name="chunk_size")
    support = _varlen_support(chunk_size, reset_chunk_pos_per_seq, position_offsets, "_flash_sca_varlen_fwd")
    with torch.no_grad():
        return varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, support, resolve_scale(q, scale))


def _flash_sca_varlen_bwd(y_grad, q, k, v, y, lse, chunk_size, scale=None, *, cu_seqlens_q, cu_seqlens_k,
                          max_seqlen_q, max_seqlen_k, position_offsets=None, backend="auto",
                          reset_chunk_pos_per_seq=False, deterministic=False, attn_method="default"):
    _resolve_attn_method(attn_method)
    validate_packed(q, k, v, chunk_size, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                    api_name="_flash_sca_varlen_bwd", span_name="chunk_size")
    support = _varlen_support(chunk_size, reset_chunk_pos_per_seq, position_offsets, "_flash_sca_varlen_bwd")
    with torch.no_grad():
        return varlen_backward(y_grad, q, k, v, y, lse, cu_seqlens_q, cu_seqlens_k, support,
                               resolve_scale(q, scale))
