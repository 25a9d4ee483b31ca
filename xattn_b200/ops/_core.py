"""One engine behind causal, sliding-window and sliding-chunk attention.

The reference routes each public op through its own autograd function and a
family of native ops chosen by window / previous-K/V / strict-past / BOS routing
(xattn/ops/_causal_attention.py:56-108,350-809, xattn/ops/sliding_chunk_attention.py:63-450).
Here every variant is the same two kernels: the variant lives in the mask plan
(one visible-key interval per query row), so dispatch reduces to building that
plan.  BOS masks become segment ids; there is no packed-varlen detour and no
host synchronisation.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _native
from . import _validation as V


@dataclass(frozen=True)
class Support:
    """Which keys left of a query are visible (tests/_reference.py:50-59)."""
    kind: str = "full"            # "full" | "window" | "chunk"
    span: Optional[int] = None    # window radius / chunk size
    reset: bool = False           # chunk positions restart per segment run
    strict: bool = False          # exclude the aligned key itself


def concat_previous(k: Tensor, v: Tensor, prev_k: Optional[Tensor], prev_v: Optional[Tensor]):
    """Total K/V = previous ‖ current (csrc/causal_attention/launch.cu:1058-1065)."""
    if prev_k is None:
        return k, v
    return torch.cat((prev_k, k), dim=1), torch.cat((prev_v, v), dim=1)


def make_plan(q: Tensor, k_length: int, support: Support,
              q_segment_idx: Optional[Tensor], k_segment_idx: Optional[Tensor]) -> Tensor:
    return _native.build_plan(
        q.shape[0], q.shape[1], k_length, q.device,
        visibility=support.kind, span=support.span, strict_past=support.strict,
        reset_positions=support.reset and q_segment_idx is not None,
        q_segment_idx=q_segment_idx, k_segment_idx=k_segment_idx,
    )


def forward(
    q: Tensor, k: Tensor, v: Tensor, support: Support, scale: float,
    prev_k: Optional[Tensor], prev_v: Optional[Tensor],
    q_segment_idx: Optional[Tensor], k_segment_idx: Optional[Tensor],
    *, high_precision: bool = False, output_state: Optional[Tensor] = None, return_plan: bool = False,
):
    """(y, lse), and the mask plan too when asked for (the autograd path keeps it for the backward)."""
    k_all, v_all = concat_previous(k, v, prev_k, prev_v)
    plan = make_plan(q, k_all.shape[1], support, q_segment_idx, k_segment_idx)
    out = _native.attention_fwd(q, k_all, v_all, plan, scale, high_precision=high_precision,
                                output_state=output_state)
    return (*out, plan) if return_plan else out


def backward(
    dy: Tensor, q: Tensor, k: Tensor, v: Tensor, y: Tensor, lse: Tensor, support: Support, scale: float,
    prev_k: Optional[Tensor], prev_v: Optional[Tensor],
    q_segment_idx: Optional[Tensor], k_segment_idx: Optional[Tensor],
    *, high_precision: bool = False, plan: Optional[Tensor] = None, recompute: bool = True,
) -> Tuple[Tensor, Tensor, Tensor, Optional[Tensor], Optional[Tensor]]:
    """(dq, dk, dv, dprev_k, dprev_v).  At level 1 the given ``y`` / ``lse`` are ignored and the
    statistics are recomputed with the high-precision softmax
    (xattn/ops/causal_flash_attn.py:144-147), unless the caller vouches that they already come from
    that forward on these inputs (``recompute=False``: the autograd path, where the recomputation
    would reproduce the saved tensors bit for bit)."""
    k_all, v_all = concat_previous(k, v, prev_k, prev_v)
    if plan is None:        # the autograd path hands over the forward's plan
        plan = make_plan(q, k_all.shape[1], support, q_segment_idx, k_segment_idx)
    if high_precision and recompute:
        y, lse = _native.attention_fwd(q, k_all, v_all, plan, scale, high_precision=True)
    dq, dk_all, dv_all = _native.attention_bwd(dy, q, k_all, v_all, y, lse, plan, scale)
    if high_precision:
        dq = _native.zero_constant_key_rows(dq, k_all, plan)
    if prev_k is None:
        return dq, dk_all, dv_all, None, None
    p = prev_k.shape[1]
    return dq, dk_all[:, p:], dv_all[:, p:], dk_all[:, :p], dv_all[:, :p]


class AttentionFunction(torch.autograd.Function):
    """Autograd bridge (the reference's _CausalAttentionFunc / _FlashSCAFunc,
    xattn/ops/_causal_attention.py:350-436, xattn/ops/sliding_chunk_attention.py:63-163)."""

    @staticmethod
    def forward(ctx, q, k, v, prev_k, prev_v, q_segment_idx, k_segment_idx, support, scale, level):
        y, lse, plan = forward(q, k, v, support, scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
                               high_precision=bool(level), return_plan=True)
        ctx.save_for_backward(q, k, v, y, lse, prev_k, prev_v, q_segment_idx, k_segment_idx, plan)
        ctx.support, ctx.scale, ctx.level = support, scale, level
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v, y, lse, prev_k, prev_v, q_seg, k_seg, plan = ctx.saved_tensors
        dq, dk, dv, dpk, dpv = backward(dy, q, k, v, y, lse, ctx.support, ctx.scale, prev_k, prev_v,
                                        q_seg, k_seg, high_precision=bool(ctx.level), plan=plan, recompute=False)
        return dq, dk, dv, dpk, dpv, None, None, None, None, None


def prepare(
    q, k, v, prev_k, prev_v, segment_idx, q_segment_idx, k_segment_idx, bos_mask, backend, *, api_name: str,
):
    """Validation common to the three op families; returns (q ids, k ids)."""
    V.normalize_backend(backend, api_name)
    prev_length = V.validate_qkv(q, k, v, prev_k, prev_v, api_name=api_name)
    _native.require_cuda(q, api_name)
    return V.resolve_segments(q, k.shape[1] + prev_length, segment_idx, q_segment_idx, k_segment_idx,
                              bos_mask, api_name=api_name)


def attention(q, k, v, support: Support, scale, prev_k, prev_v, q_segment_idx, k_segment_idx, *,
              segment_idx, bos_mask, backend, deterministic, high_precision_level, api_name) -> Tensor:
    if not isinstance(deterministic, bool):
        raise TypeError(f"{api_name} deterministic must be a bool")
    q_ids, k_ids = prepare(q, k, v, prev_k, prev_v, segment_idx, q_segment_idx, k_segment_idx, bos_mask,
                           backend, api_name=api_name)
    return AttentionFunction.apply(q, k, v, prev_k, prev_v, q_ids, k_ids, support,
                                   V.resolve_scale(q, scale), high_precision_level)


def attention_fwd(q, k, v, support: Support, scale, prev_k, prev_v, q_segment_idx, k_segment_idx, *,
                  segment_idx, bos_mask, backend, high_precision_level, api_name) -> Tuple[Tensor, Tensor]:
    q_ids, k_ids = prepare(q, k, v, prev_k, prev_v, segment_idx, q_segment_idx, k_segment_idx, bos_mask,
                           backend, api_name=api_name)
    with torch.no_grad():
        return forward(q, k, v, support, V.resolve_scale(q, scale), prev_k, prev_v, q_ids, k_ids,
                       high_precision=bool(high_precision_level))


def attention_bwd(y_grad, q, k, v, y, lse, support: Support, scale, prev_k, prev_v, q_segment_idx,
                  k_segment_idx, *, segment_idx, bos_mask, backend, deterministic, high_precision_level,
                  api_name):
    V.validate_attention_output(y, q)
    if not isinstance(deterministic, bool):
        raise TypeError(f"{api_name} deterministic must be a bool")
    q_ids, k_ids = prepare(q, k, v, prev_k, prev_v, segment_idx, q_segment_idx, k_segment_idx, bos_mask,
                           backend, api_name=api_name)
    V.validate_saved_state(y, lse, q, v)
    if y_grad.shape != y.shape or y_grad.dtype != q.dtype or y_grad.device != q.device:
        raise ValueError(f"{api_name} y_grad must match y in shape, dtype and device")
    with torch.no_grad():
        return backward(y_grad, q, k, v, y, lse, support, V.resolve_scale(q, scale), prev_k, prev_v,
                        q_ids, k_ids, high_precision=bool(high_precision_level))
