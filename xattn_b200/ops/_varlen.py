"""Packed variable-length inputs ``[T, H, D]`` with cu_seqlens.

The reference has dedicated varlen native ops (csrc/causal_attention/launch.cu:1455-1695,
xattn/ops/_varlen_metadata.py:1-97).  Here a packed batch is one batch row whose plan encodes the
sequence boundaries, so the same kernels run.  lse comes back as ``[H, T]`` like the reference's.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _native

_INT32_MAX = 2**31 - 1


def validate_packed(q, k, v, span, cu_q, cu_k, max_q, max_k, *, api_name: str, span_name: str) -> None:
    if span is not None:
        if isinstance(span, bool) or not isinstance(span, int):
            raise TypeError(f"{api_name} {span_name} must be an integer")
        if span < 0 or (span_name == "chunk_size" and span == 0):
            raise ValueError(f"{api_name} {span_name} must be " + ("positive" if span_name == "chunk_size" else "nonnegative"))
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError(f"{api_name} expects packed 3D q/k/v tensors")
    if q.device != k.device or q.device != v.device:
        raise ValueError(f"{api_name} q/k/v must be on the same device")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError(f"{api_name} q/k/v must have the same dtype")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"{api_name} supports only torch.float16 and torch.bfloat16 input; got {q.dtype}")
    if k.shape[0] != v.shape[0]:
        raise ValueError(f"{api_name} packed k/v token counts must match")
    if k.shape[1] != v.shape[1]:
        raise ValueError(f"{api_name} k/v head counts must match")
    if q.shape[1] <= 0 or k.shape[1] <= 0:
        raise ValueError(f"{api_name} q and kv head counts must be positive")
    if q.shape[1] % k.shape[1] != 0:
        raise ValueError(f"{api_name} q head count must be divisible by kv head count; got Hq={q.shape[1]}, Hkv={k.shape[1]}")
    if q.shape[2] != k.shape[2]:
        raise ValueError(f"{api_name} q/k head dims must match")
    if q.shape[2] <= 0 or v.shape[2] <= 0:
        raise ValueError(f"{api_name} q/k and value head dims must be positive")
    if cu_q.dim() != 1 or cu_k.dim() != 1:
        raise ValueError(f"{api_name} cu_seqlens_q/cu_seqlens_k must be 1D")
    if cu_q.dtype != torch.int32 or cu_k.dtype != torch.int32:
        raise ValueError(f"{api_name} cu_seqlens must be torch.int32")
    if cu_q.device != q.device or cu_k.device != q.device:
        raise ValueError(f"{api_name} cu_seqlens must share the Q/K/V device")
    if cu_q.numel() < 2:
        raise ValueError(f"{api_name} cu_seqlens must contain at least one sequence")
    if cu_k.numel() < cu_q.numel():
        raise ValueError(f"{api_name} right-aligned varlen requires at least as many K sequences as Q sequences")
    for name, value in (("max_seqlen_q", max_q), ("max_seqlen_k", max_k)):
        if isinstance(value, bool) or not isinstance(value, int):
            raise TypeError(f"{api_name} max_seqlen_q/max_seqlen_k must be integers")
        if value <= 0:
            raise ValueError(f"{api_name} max_seqlen_q/max_seqlen_k must be positive")
    if q.shape[0] > _INT32_MAX or k.shape[0] > _INT32_MAX:
        raise ValueError(f"{api_name} varlen sizes must fit int32")


def _plan(q, k, cu_q, cu_k, support):
    return _native.build_varlen_plan(cu_q, cu_k, q.shape[0], k.shape[0], visibility=support.kind,
                                     span=support.span, strict_past=support.strict)


def varlen_forward(q, k, v, cu_q, cu_k, support, scale, *, output_state: Optional[Tensor] = None,
                   high_precision: bool = False) -> Tuple[Tensor, Tensor]:
    _native.require_cuda(q, "packed varlen attention")
    if q.shape[0] == 0:
        return q.new_empty((0, q.shape[1], v.shape[2])), q.new_empty((q.shape[1], 0), dtype=torch.float32)
    plan = _plan(q, k, cu_q, cu_k, support)
    state = None if output_state is None else output_state.unsqueeze(0)
    y, lse = _native.attention_fwd(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), plan, scale,
                                   high_precision=high_precision, output_state=state)
    return y.squeeze(0), lse.squeeze(0)


def varlen_backward(dy, q, k, v, y, lse, cu_q, cu_k, support, scale):
    if q.shape[0] == 0:
        return torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    plan = _plan(q, k, cu_q, cu_k, support)
    dq, dk, dv = _native.attention_bwd(dy.unsqueeze(0), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0),
                                       y.unsqueeze(0), lse.unsqueeze(0), plan, scale)
    return dq.squeeze(0), dk.squeeze(0), dv.squeeze(0)


class VarlenFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, support, scale):
        y, lse = varlen_forward(q, k, v, cu_q, cu_k, support, scale)
        ctx.save_for_backward(q, k, v, y, lse, cu_q, cu_k)
        ctx.support, ctx.scale = support, scale
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v, y, lse, cu_q, cu_k = ctx.saved_tensors
        dq, dk, dv = varlen_backward(dy, q, k, v, y, lse, cu_q, cu_k, ctx.support, ctx.scale)
        return dq, dk, dv, None, None, None, None
