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

import os
import threading
from collections import OrderedDict
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


class _PlanCache(threading.local):
    """Mask plans (and the segment ids of BOS masks) of recent calls, per thread.

    The reference keeps a thread-local cache of its sliding-chunk forward plan for inference with
    repeated BOS masks, keyed by tensor identity and stream
    (csrc/flash_sca/sliding_chunk_attention.cc:113-518, xattn/ops/sliding_chunk_attention.py:2163-2297),
    because building that plan synchronises with the host.  The plan here is built on the device, so
    the cache only saves its three to five small kernels (and the running sum over a BOS mask): what
    matters for decode-sized calls, where they cost as much as the attention itself.

    * A dense plan (no segment metadata) depends on nothing but the shapes and the visibility rule: it
      is cached for every call (per stream, like every entry: a plan is ready in the order of the stream
      that built it).
    * A plan built from segment ids or a BOS mask is keyed by the identity of the metadata tensor
      (storage address, offset, shape, strides, version counter) and the current stream; the entry
      holds the tensor, so its memory cannot be handed to another tensor meanwhile, and a write into
      the mask changes its version.  Tensors created under inference mode have no version counter:
      after writing into such a mask in place, call ``clear_plan_cache()``.  A training loop whose
      masks change every step only cycles the cache's sixteen entries.
    * Nothing is stored while a CUDA graph is being captured (memory of the capture's private pool
      must not outlive it); lookups still work.
    ``XATTN_B200_PLAN_CACHE=0`` disables it."""

    CAPACITY = 16

    def __init__(self):
        self.entries: "OrderedDict[tuple, tuple]" = OrderedDict()
        self.hits = 0
        self.misses = 0

    def get(self, key):
        hit = self.entries.get(key)
        if hit is None:
            self.misses += 1
            return None
        self.entries.move_to_end(key)
        self.hits += 1
        return hit

    def put(self, key, value):
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            return
        self.entries[key] = value
        while len(self.entries) > self.CAPACITY:
            self.entries.popitem(last=False)


_plan_cache = _PlanCache()


def plan_cache_enabled() -> bool:
    return os.environ.get("XATTN_B200_PLAN_CACHE", "1") != "0"


def clear_plan_cache() -> None:
    """Drop every cached plan of the calling thread (the reference's
    ``_flash_sca_sm90_clear_inference_bos_fwd_plan_cache``)."""
    _plan_cache.entries.clear()


def plan_cache_stats() -> Tuple[int, int]:
    """(hits, misses) of the calling thread since start."""
    return _plan_cache.hits, _plan_cache.misses


def _identity(t: Optional[Tensor]):
    """What makes a metadata tensor 'the same tensor with the same contents' for the cache."""
    if t is None:
        return None
    try:
        version = t._version
    except RuntimeError:            # inference tensors do not count their writes
        version = -1
    return (t.data_ptr(), t.storage_offset(), tuple(t.shape), tuple(t.stride()), t.dtype, version)


def make_plan(q: Tensor, k_length: int, support: Support,
              q_segment_idx: Optional[Tensor], k_segment_idx: Optional[Tensor]) -> Tensor:
    use_cache = plan_cache_enabled() and q.is_cuda
    key = None
    if use_cache:
        key = ("plan", q.device, q.shape[0], q.shape[1], k_length, support, _identity(q_segment_idx),
               _identity(k_segment_idx), torch.cuda.current_stream(q.device).cuda_stream)
        hit = _plan_cache.get(key)
        if hit is not None:
            return hit[0]
    plan = _native.build_plan(
        q.shape[0], q.shape[1], k_length, q.device,
        visibility=support.kind, span=support.span, strict_past=support.strict,
        reset_positions=support.reset and q_segment_idx is not None,
        q_segment_idx=q_segment_idx, k_segment_idx=k_segment_idx,
    )
    if use_cache:
        _plan_cache.put(key, (plan, q_segment_idx, k_segment_idx))      # the ids stay alive with the entry
    return plan


def forward(
    q: Tensor, k: Tensor, v: Tensor, support: Support, scale: float,
    prev_k: Optional[Tensor], prev_v: Optional[Tensor],
    q_segment_idx: Optional[Tensor], k_segment_idx: Optional[Tensor],
    *, high_precision: bool = False, output_state: Optional[Tensor] = None, return_plan: bool = False,
):
    """(y, lse), and with ``return_plan`` (the autograd path, which keeps them for the backward) the mask
    plan and, at level 1, the rows' anchor keys too (``None`` at level 0)."""
    k_all, v_all = concat_previous(k, v, prev_k, prev_v)
    plan = make_plan(q, k_all.shape[1], support, q_segment_idx, k_segment_idx)
    out = _native.attention_fwd(q, k_all, v_all, plan, scale, high_precision=high_precision,
                                output_state=output_state, return_anchor=return_plan and high_precision)
    if not return_plan:
        return out
    return (*out, plan) if high_precision else (*out, None, plan)


def prescale_fp16(dy: Tensor, v_all: Tensor):
    """Level 1, FP16 only: ``dy`` times a power of two that keeps dS = P (dP - delta), bounded by
    2 max|dO_i| max|V_j|, near 2^13 and so out of the FP16 subnormals, and the FP32 device scalar that
    undoes it on the gradients (gradients are linear in ``dy``, so both steps are exact).  Restates
    xattn/ops/_precision_backend.py:203-225; stays on the device, no synchronisation."""
    if dy.dtype != torch.float16 or not dy.numel() or not v_all.numel():
        return dy, None
    g = torch.linalg.vector_norm(dy, dim=-1, dtype=torch.float32).amax()
    w = torch.linalg.vector_norm(v_all, dim=-1, dtype=torch.float32).amax()
    bound = 2 * g * w
    e = torch.floor(torch.log2(2.0 ** 13 / bound))
    e = torch.minimum(e, torch.floor(torch.log2(30000.0 / dy.abs().amax().float())))   # dy stays finite
    e = torch.where(bound > 32768.0, e, e.clamp_min(0))
    e = torch.where(torch.isfinite(e), e, torch.zeros_like(e)).clamp(-60, 60).to(torch.int32)
    factor = ((e + 127) << 23).view(torch.float32)
    return (dy.float() * factor).to(dy.dtype), ((127 - e) << 23).view(torch.float32).reshape(1)


def backward(
    dy: Tensor, q: Tensor, k: Tensor, v: Tensor, y: Tensor, lse: Tensor, support: Support, scale: float,
    prev_k: Optional[Tensor], prev_v: Optional[Tensor],
    q_segment_idx: Optional[Tensor], k_segment_idx: Optional[Tensor],
    *, high_precision: bool = False, plan: Optional[Tensor] = None, anchor: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor, Tensor, Optional[Tensor], Optional[Tensor]]:
    """(dq, dk, dv, dprev_k, dprev_v).  Level 1 is the anchored backward of ``_native.attention_bwd``
    followed by the exact zeroing of dQ rows whose visible keys are one repeated vector.  It needs the
    statistics of the high-precision forward: the given ``y`` / ``lse`` are ignored and the forward is
    run again (xattn/ops/causal_flash_attn.py:144-147), unless the caller hands over that forward's
    own ``lse`` and ``anchor`` (the autograd path)."""
    k_all, v_all = concat_previous(k, v, prev_k, prev_v)
    if plan is None:        # the autograd path hands over the forward's plan
        plan = make_plan(q, k_all.shape[1], support, q_segment_idx, k_segment_idx)
    if high_precision:
        if anchor is None:
            y, lse, anchor = _native.attention_fwd(q, k_all, v_all, plan, scale, high_precision=True,
                                                   return_anchor=True)
        dy, unscale = prescale_fp16(dy, v_all)
        dq, dk_all, dv_all = _native.attention_bwd(dy, q, k_all, v_all, y, lse, plan, scale, anchor=anchor,
                                                   grad_unscale=unscale)
        dq = _native.zero_constant_key_rows(dq, k_all, plan)
    else:
        dq, dk_all, dv_all = _native.attention_bwd(dy, q, k_all, v_all, y, lse, plan, scale)
    if prev_k is None:
        return dq, dk_all, dv_all, None, None
    p = prev_k.shape[1]
    return dq, dk_all[:, p:], dv_all[:, p:], dk_all[:, :p], dv_all[:, :p]


class AttentionFunction(torch.autograd.Function):
    """Autograd bridge (the reference's _CausalAttentionFunc / _FlashSCAFunc,
    xattn/ops/_causal_attention.py:350-436, xattn/ops/sliding_chunk_attention.py:63-163)."""

    @staticmethod
    def forward(ctx, q, k, v, prev_k, prev_v, q_segment_idx, k_segment_idx, support, scale, level):
        y, lse, anchor, plan = forward(q, k, v, support, scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
                                       high_precision=bool(level), return_plan=True)
        ctx.save_for_backward(q, k, v, y, lse, prev_k, prev_v, q_segment_idx, k_segment_idx, plan, anchor)
        ctx.support, ctx.scale, ctx.level = support, scale, level
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v, y, lse, prev_k, prev_v, q_seg, k_seg, plan, anchor = ctx.saved_tensors
        dq, dk, dv, dpk, dpv = backward(dy, q, k, v, y, lse, ctx.support, ctx.scale, prev_k, prev_v,
                                        q_seg, k_seg, high_precision=bool(ctx.level), plan=plan, anchor=anchor)
        return dq, dk, dv, dpk, dpv, None, None, None, None, None


def prepare(
    q, k, v, prev_k, prev_v, segment_idx, q_segment_idx, k_segment_idx, bos_mask, backend, *, api_name: str,
):
    """Validation common to the three op families; returns (q ids, k ids)."""
    V.normalize_backend(backend, api_name)
    prev_length = V.validate_qkv(q, k, v, prev_k, prev_v, api_name=api_name)
    _native.require_cuda(q, api_name)
    return resolve_segments_cached(q, k.shape[1] + prev_length, segment_idx, q_segment_idx, k_segment_idx,
                                   bos_mask, api_name=api_name)


def resolve_segments_cached(q, k_length, segment_idx, q_segment_idx, k_segment_idx, bos_mask, *, api_name):
    """``_validation.resolve_segments``, with the ids of a BOS mask seen before taken from the plan cache:
    the same id tensors come back, so the plan built from them is found again too."""
    only_bos = bos_mask is not None and segment_idx is None and q_segment_idx is None and k_segment_idx is None
    if not (only_bos and isinstance(bos_mask, Tensor) and bos_mask.is_cuda and plan_cache_enabled()):
        return V.resolve_segments(q, k_length, segment_idx, q_segment_idx, k_segment_idx, bos_mask, api_name=api_name)
    key = ("bos", q.device, q.shape[0], q.shape[1], k_length, _identity(bos_mask),
           torch.cuda.current_stream(q.device).cuda_stream)
    hit = _plan_cache.get(key)
    if hit is not None:
        return hit[0], hit[1]
    ids = V.resolve_segments(q, k_length, None, None, None, bos_mask, api_name=api_name)
    _plan_cache.put(key, (ids[0], ids[1], bos_mask))
    return ids


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
