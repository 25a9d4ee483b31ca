"""SoftDelta attention: a gated negative read shared by each KV group.

Per query head ``h`` with KV head ``kv(h)`` (xattn/ops/softdelta_attention.py:3-29)::

    read_h      = Attention(q_h,       K, V; inclusive causal support)
    neg_read_kv = Attention(k_read_kv, K, V; strict-past causal support)
    y_h         = read_h - sigmoid(g_h) * neg_read_kv(h)

The reference fuses both reads into one Hopper launch over "logical heads"
(csrc/softdelta/fwd.cu:143-231) and has a fused backward (csrc/softdelta/bwd.cu:99-239).  Here
both reads are launches of the same forward kernel — the strict-past read is just another mask
plan — followed by one gate kernel; the backward is the gate kernel's backward pass followed
by two launches of the attention backward, with the aligned keys' query-side gradient folded
into ``dk`` when ``k_read`` is None.  ``backend='torch'`` is the reference's pure-torch
correctness plan (xattn/ops/softdelta_attention.py:571-620) and works on any device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _native
from . import _core
from ._validation import (dispatch_nonpositive_scale, resolve_scale, resolve_segments,
                          validate_attention_scale, validate_chunk_size, validate_dimensions,
                          validate_gate_and_reader, validate_high_precision_level, validate_qkv,
                          validate_window_size)

__all__ = [
    "softdelta_attention", "softdelta_attention_fwd", "softdelta_attention_bwd",
    "sliding_window_softdelta_attention", "sliding_window_softdelta_attention_fwd",
    "sliding_window_softdelta_attention_bwd",
    "sliding_chunk_softdelta_attention", "sliding_chunk_softdelta_attention_fwd",
    "sliding_chunk_softdelta_attention_bwd",
]


def _normalize_backend(backend) -> str:
    if not isinstance(backend, str):
        raise TypeError("SoftDelta backend must be a string")
    name = backend.strip().lower().replace("-", "_")
    if name not in ("", "auto", "torch", "sm90", "sm100", "sm100a"):
        raise ValueError("SoftDelta backend must be one of: auto, torch, sm90, sm100")
    return "auto" if name == "" else name


def _validate(q, k, v, g, k_read, prev_k, prev_v, deterministic, api_name) -> int:
    """The shared q/k/v (+ previous K/V) contract, then the gate and the second reader; returns the
    previous-K/V length."""
    prev_length = validate_qkv(q, k, v, prev_k, prev_v, api_name=api_name)
    validate_gate_and_reader(q, k, g, k_read, deterministic, api_name=api_name)
    return prev_length


def _support(kind: str, a: dict, api_name: str) -> _core.Support:
    if kind == "full":
        return _core.Support("full")
    if kind == "window":
        validate_window_size(a["window_size"], api_name)
        return _core.Support("window", a["window_size"])
    validate_chunk_size(a["chunk_size"], api_name)
    reset = a["reset_chunk_pos_per_seq"]
    if not isinstance(reset, bool):
        raise TypeError(f"{api_name} reset_chunk_pos_per_seq must be a bool")
    prev_k = a.get("prev_k")
    if prev_k is not None and prev_k.dim() == 4 and prev_k.shape[1] != a["chunk_size"]:
        raise ValueError(f"{api_name} prev_k/prev_v sequence length must equal chunk_size")
    return _core.Support("chunk", a["chunk_size"], reset)


def _aligned_keys(k: Tensor, q_length: int) -> Tensor:
    return k if k.shape[1] == q_length else k[:, k.shape[1] - q_length:]


def _strict(s: _core.Support) -> _core.Support:
    return _core.Support(s.kind, s.span, s.reset, True)


# ---- the three compute plans ---------------------------------------------------------------------

def _forward(q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, scale, level, support):
    """(y, neg_read, lse, read_lse_offset): two reads and the gate."""
    k_all, v_all = _core.concat_previous(k, v, prev_k, prev_v)
    kr = _aligned_keys(k, q.shape[1]) if k_read is None else k_read
    plan_inc = _core.make_plan(q, k_all.shape[1], support, q_ids, k_ids)
    plan_strict = _core.make_plan(q, k_all.shape[1], _strict(support), q_ids, k_ids)
    hp = bool(level)
    read, lse_read = _native.attention_fwd(q, k_all, v_all, plan_inc, scale, high_precision=hp)
    neg_state = None
    if hp:
        neg_state = torch.empty((*kr.shape[:3], v.shape[3]), dtype=torch.float32, device=q.device)
    neg, lse_neg = _native.attention_fwd(kr, k_all, v_all, plan_strict, scale, high_precision=hp,
                                         output_state=neg_state)
    neg_read = neg_state if hp else neg
    y = _native.softdelta_gate_fwd(read, neg_read, g, out=read)
    return y, neg_read, torch.cat((lse_neg, lse_read), dim=1)


def _backward(dy, q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, y, neg_read, lse, scale, level, support):
    """(dq, dk, dv, dg, dk_read, dprev_k, dprev_v)."""
    k_all, v_all = _core.concat_previous(k, v, prev_k, prev_v)
    L, Hkv = q.shape[1], k.shape[2]
    kr = _aligned_keys(k, L) if k_read is None else k_read
    plan_inc = _core.make_plan(q, k_all.shape[1], support, q_ids, k_ids)
    plan_strict = _core.make_plan(q, k_all.shape[1], _strict(support), q_ids, k_ids)
    hp = bool(level)
    read, dneg, dg = _native.softdelta_gate_bwd(dy, y, neg_read, g)
    lse_neg, lse_read = lse[:, :Hkv], lse[:, Hkv:]
    neg = neg_read if neg_read.dtype == q.dtype else neg_read.to(q.dtype)
    if hp:
        # level 1 recomputes the statistics of both reads with the high-precision softmax, takes their
        # anchor keys along and runs the anchored backward on each read
        read, lse_read, a_read = _native.attention_fwd(q, k_all, v_all, plan_inc, scale, high_precision=True,
                                                       return_anchor=True)
        neg, lse_neg, a_neg = _native.attention_fwd(kr, k_all, v_all, plan_strict, scale, high_precision=True,
                                                    return_anchor=True)
        dy1, un1 = _core.prescale_fp16(dy, v_all)
        dy2, un2 = _core.prescale_fp16(dneg, v_all)
        dq, dk1, dv1 = _native.attention_bwd(dy1, q, k_all, v_all, read, lse_read, plan_inc, scale,
                                             anchor=a_read, grad_unscale=un1)
        dkr, dk2, dv2 = _native.attention_bwd(dy2, kr, k_all, v_all, neg, lse_neg, plan_strict, scale,
                                              anchor=a_neg, grad_unscale=un2)
    else:
        dq, dk1, dv1 = _native.attention_bwd(dy, q, k_all, v_all, read, lse_read, plan_inc, scale)
        dkr, dk2, dv2 = _native.attention_bwd(dneg, kr, k_all, v_all, neg, lse_neg, plan_strict, scale)
    if hp:
        dq = _native.zero_constant_key_rows(dq, k_all, plan_inc)
        dkr = _native.zero_constant_key_rows(dkr, k_all, plan_strict)
    # FP32 sums rounded once; the aligned keys' own gradient folds into the last L rows of dK
    dk_all = _native.softdelta_merge_gradients(dk1, dk2, dkr if k_read is None else None)
    dv_all = _native.softdelta_merge_gradients(dv1, dv2)
    dk_read = None if k_read is None else dkr
    if prev_k is None:
        return dq, dk_all, dv_all, dg, dk_read, None, None
    p = prev_k.shape[1]
    return dq, dk_all[:, p:], dv_all[:, p:], dg, dk_read, dk_all[:, :p], dv_all[:, :p]


def _torch_plan(q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, scale, support):
    """Pure-torch correctness plan (FP32 accumulation), differentiable by autograd; any device."""
    k_all, v_all = _core.concat_previous(k, v, prev_k, prev_v)
    B, L, H, _ = q.shape
    Lk, Hkv = k_all.shape[1], k_all.shape[2]
    kr = _aligned_keys(k, L) if k_read is None else k_read
    dev = q.device
    if q_ids is None:
        same = torch.ones(B, L, Lk, dtype=torch.bool, device=dev)
        q_pos = (torch.arange(L, device=dev) + (Lk - L)).expand(B, L)
        k_pos = torch.arange(Lk, device=dev).expand(B, Lk)
    else:
        same = q_ids[:, :, None] == k_ids[:, None, :]
        if support.reset:
            def runs(ids):
                n = ids.shape[1]
                pos = torch.arange(n, device=dev).expand_as(ids)
                first = torch.ones_like(ids, dtype=torch.bool)
                last = torch.ones_like(ids, dtype=torch.bool)
                if n > 1:
                    ch = ids[:, 1:] != ids[:, :-1]
                    first[:, 1:] = ch
                    last[:, :-1] = ch
                start = torch.where(first, pos, torch.zeros_like(pos)).cummax(1).values
                end = torch.where(last, pos + 1, torch.full_like(pos, n)).flip(1).cummin(1).values.flip(1)
                return pos - start, end - start
            q_local, q_run = runs(q_ids)
            k_pos, _ = runs(k_ids)
            q_pos = q_local + same.sum(-1) - q_run
        else:
            q_pos = (torch.arange(L, device=dev) + (Lk - L)).expand(B, L)
            k_pos = torch.arange(Lk, device=dev).expand(B, Lk)
    qp, kp = q_pos[:, :, None], k_pos[:, None, :]
    left = torch.ones_like(same)
    if support.kind == "window":
        left = kp >= qp - support.span
    elif support.kind == "chunk":
        left = kp >= torch.div(qp, support.span, rounding_mode="floor") * support.span - support.span
    inclusive = same & left & (kp <= qp)
    strict = same & left & (kp < qp)

    def read(query, allowed):
        rep = query.shape[2] // Hkv
        kk = k_all.repeat_interleave(rep, 2) if rep != 1 else k_all
        vv = v_all.repeat_interleave(rep, 2) if rep != 1 else v_all
        acc = torch.float64 if query.dtype == torch.float64 else torch.float32
        s = torch.einsum("bqhd,bkhd->bhqk", query.to(acc), kk.to(acc)) * scale
        keep = allowed[:, None]
        s = s.masked_fill(~keep, float("-inf"))
        s = torch.where(allowed.any(-1, keepdim=True)[:, None], s, torch.zeros_like(s))
        p = torch.softmax(s, -1).masked_fill(~keep, 0.0)
        return torch.einsum("bhqk,bkhv->bqhv", p, vv.to(acc))

    r = read(q, inclusive)
    n = read(kr, strict)
    rep = H // Hkv
    gate = torch.sigmoid(g.to(r.dtype)).view(B, L, Hkv, rep, 1)
    y = r.view(B, L, Hkv, rep, -1) - gate * n[:, :, :, None, :]
    return y.reshape(B, L, H, -1).to(g.dtype)


class _SoftDeltaFunction(torch.autograd.Function):
    """Scalar gates (the public layout: ``v`` [B, L, Hkv, V], ``g`` [B, Lq, H]) or the reference's internal
    value groups (``v`` [B, L, Hkv, C, Dg], ``g`` [B, Lq, H, C, 1], one gate per group of ``Dg`` channels:
    xattn/ops/softdelta_attention.py ``_SoftDeltaFunc``, tests/softdelta/test_value_groups.py:1-7).  Both
    reads are linear in V, so the grouped form runs them on the flattened values and differs only in the
    gate kernel; outputs and gradients follow the input layout."""

    @staticmethod
    def forward(ctx, q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, scale, level, support):
        groups = None
        if v.dim() == 5:
            groups = tuple(v.shape[3:])
            if g.shape != (*q.shape[:3], groups[0], 1):
                raise ValueError("grouped SoftDelta expects g of shape [B, Lq, H, C, 1]")
            v = v.flatten(3)
            prev_v = None if prev_v is None else prev_v.flatten(3)
            g = g.squeeze(-1)
        y, neg_read, lse = _forward(q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, scale, level, support)
        ctx.save_for_backward(q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, y, neg_read, lse)
        ctx.scale, ctx.level, ctx.support, ctx.groups = scale, level, support, groups
        return y if groups is None else y.unflatten(3, groups)

    @staticmethod
    def backward(ctx, dy):
        q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, y, neg_read, lse = ctx.saved_tensors
        groups = ctx.groups
        if groups is not None:
            dy = dy.flatten(3)
        dq, dk, dv, dg, dk_read, dpk, dpv = _backward(
            dy, q, k, v, g, k_read, prev_k, prev_v, q_ids, k_ids, y, neg_read, lse,
            ctx.scale, ctx.level, ctx.support)
        if groups is not None:
            dv = dv.unflatten(3, groups)
            dg = dg.unsqueeze(-1)
            dpv = None if dpv is None else dpv.unflatten(3, groups)
        return dq, dk, dv, dg, dk_read, dpk, dpv, None, None, None, None, None


def _softdelta_value_groups(q, k, v, g, k_read=None, *, scale=None, q_segment_idx=None, k_segment_idx=None,
                            visibility="full", span=None, high_precision_level=0):
    """Internal entry for the value-group layout (no public API takes it yet, as in the reference):
    ``v`` [B, L, Hkv, C, Dg], ``g`` [B, Lq, H, C, 1]; ``visibility`` full / window / chunk with ``span``."""
    if v.dim() != 5 or g.dim() != 5:
        raise ValueError("value-group SoftDelta expects 5D v and g")
    support = _core.Support(visibility, span, False, False)
    resolved = q.shape[-1] ** -0.5 if scale is None else float(scale)
    return _SoftDeltaFunction.apply(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(),
                                    None if k_read is None else k_read.contiguous(), None, None,
                                    q_segment_idx, k_segment_idx, resolved, int(high_precision_level), support)


# ---- shared call paths --------------------------------------------------------------------------

def _prepare(fn, kind, a, standalone):
    name = fn.__name__
    level = validate_high_precision_level(a["high_precision_level"], api_name=name)
    validate_dimensions(a["q"], a["v"], a["backend"], api_name=name)
    backend = _normalize_backend(a["backend"])
    q, k, v, g, k_read = a["q"], a["k"], a["v"], a["g"], a["k_read"]
    prev_k, prev_v = a.get("prev_k"), a.get("prev_v")
    prev_length = _validate(q, k, v, g, k_read, prev_k, prev_v, a["deterministic"], name)
    support = _support(kind, a, name)
    use_native = backend != "torch" and q.is_cuda
    if backend in ("sm90", "sm100", "sm100a") or (standalone and backend != "torch"):
        _native.require_cuda(q, name)
    if standalone and backend == "torch":
        raise RuntimeError(f"{name} needs the CUDA kernels; backend='torch' only serves the autograd call")
    q_ids, k_ids = resolve_segments(q, k.shape[1] + prev_length, a["segment_idx"], a["q_segment_idx"],
                                    a["k_segment_idx"], a["bos_mask"], api_name=name)
    return (q, k, v, g, k_read, prev_k, prev_v), q_ids, k_ids, resolve_scale(q, a["scale"]), level, support, use_native


def _call(fn, kind, a):
    if a["scale"] is not None and float(a["scale"]) <= 0:
        return dispatch_nonpositive_scale(fn, a)
    tensors, q_ids, k_ids, scale, level, support, use_native = _prepare(fn, kind, a, standalone=False)
    if not use_native:
        return _torch_plan(*tensors, q_ids, k_ids, scale, support)
    return _SoftDeltaFunction.apply(*tensors, q_ids, k_ids, scale, level, support)


def _call_fwd(fn, kind, a):
    if a["scale"] is not None and float(a["scale"]) <= 0:
        return dispatch_nonpositive_scale(fn, a)
    tensors, q_ids, k_ids, scale, level, support, _ = _prepare(fn, kind, a, standalone=True)
    return _forward(*tensors, q_ids, k_ids, scale, level, support)


def _call_bwd(fn, kind, a):
    if a["scale"] is not None and float(a["scale"]) <= 0:
        return dispatch_nonpositive_scale(fn, a)
    tensors, q_ids, k_ids, scale, level, support, _ = _prepare(fn, kind, a, standalone=True)
    q, k, v, g, k_read, prev_k, prev_v = tensors
    y_grad, y, neg_read, lse = (a[n] for n in ("y_grad", "y", "neg_read", "lse"))
    B, L, H, _ = q.shape
    Hkv, V = k.shape[2], v.shape[-1]
    for nm, t, shape, dtype in (
        ("y_grad", y_grad, (B, L, H, V), q.dtype),
        ("y", y, (B, L, H, V), q.dtype),
        ("neg_read", neg_read, (B, L, Hkv, V), torch.float32 if level else q.dtype),
        ("lse", lse, (B, Hkv + H, L), torch.float32),
    ):
        if tuple(t.shape) != shape or t.device != q.device or t.dtype != dtype:
            raise ValueError(f"{fn.__name__} {nm} has incompatible shape, device, or dtype")
    dq, dk, dv, dg, dk_read, dpk, dpv = _backward(y_grad, *tensors, q_ids, k_ids, y, neg_read, lse,
                                                  scale, level, support)
    grads = (dq, dk, dv, dg, dk_read)
    return grads if "prev_k" not in a else (*grads, dpk, dpv)


# ---- public ops (signatures of xattn/ops/softdelta_attention.py:798-1065) ----------------------------

def softdelta_attention(q, k, k_read, v, g, scale=None, q_segment_idx=None, k_segment_idx=None, *,
                        segment_idx=None, bos_mask=None, backend="auto", deterministic=False,
                        high_precision_level=0) -> Tensor:
    """Causal SoftDelta attention with autograd.

    ``q`` ``[B, Lq, H, D]``, ``k`` ``[B, Lkv, Hkv, D]``, ``v`` ``[B, Lkv, Hkv, V]``, gate logits ``g``
    ``[B, Lq, H]``; ``Lq <= Lkv``, ``H % Hkv == 0``; query ``i`` aligns to key ``i + Lkv - Lq``.  The
    output ``[B, Lq, H, V]`` is ``read - sigmoid(g) * neg_read``: ``read`` covers every visible key
    up to and including the aligned one, ``neg_read`` only strictly earlier keys, once per KV head,
    queried by ``k_read`` ``[B, Lq, Hkv, D]`` (``None``: the aligned keys, whose query-side gradient
    is then added to ``dk``).  ``neg_read`` is zero on rows without an earlier visible key.
    """
    validate_attention_scale(scale)
    return _call(softdelta_attention, "full", locals())


@torch.no_grad()
def softdelta_attention_fwd(q, k, k_read, v, g, scale=None, q_segment_idx=None, k_segment_idx=None, *,
                            segment_idx=None, bos_mask=None, backend="auto", deterministic=False,
                            high_precision_level=0) -> Tuple[Tensor, Tensor, Tensor]:
    """``(y, neg_read, lse)``: ``neg_read`` ``[B, Lq, Hkv, V]`` in the input dtype (FP32 at level 1),
    ``lse`` FP32 ``[B, Hkv + H, Lq]`` with the negative reads first."""
    validate_attention_scale(scale)
    return _call_fwd(softdelta_attention_fwd, "full", locals())


@torch.no_grad()
def softdelta_attention_bwd(y_grad, q, k, k_read, v, g, y, neg_read, lse, scale=None, q_segment_idx=None,
                            k_segment_idx=None, *, segment_idx=None, bos_mask=None, backend="auto",
                            deterministic=False, high_precision_level=0):
    """``(dq, dk, dv, dg, dk_read)``; ``dk_read`` is None when ``k_read`` is."""
    validate_attention_scale(scale)
    return _call_bwd(softdelta_attention_bwd, "full", locals())


def sliding_window_softdelta_attention(q, k, k_read, v, g, window_size, scale=None, q_segment_idx=None,
                                       k_segment_idx=None, *, segment_idx=None, bos_mask=None,
                                       backend="auto", deterministic=False, high_precision_level=0) -> Tensor:
    """SoftDelta within a causal sliding window: the query read sees ``[i - window_size, i]``, the
    negative read ``[i - window_size, i - 1]``."""
    validate_attention_scale(scale)
    return _call(sliding_window_softdelta_attention, "window", locals())


@torch.no_grad()
def sliding_window_softdelta_attention_fwd(q, k, k_read, v, g, window_size, scale=None, q_segment_idx=None,
                                           k_segment_idx=None, *, segment_idx=None, bos_mask=None,
                                           backend="auto", deterministic=False, high_precision_level=0):
    validate_attention_scale(scale)
    return _call_fwd(sliding_window_softdelta_attention_fwd, "window", locals())


@torch.no_grad()
def sliding_window_softdelta_attention_bwd(y_grad, q, k, k_read, v, g, y, neg_read, lse, window_size,
                                           scale=None, q_segment_idx=None, k_segment_idx=None, *,
                                           segment_idx=None, bos_mask=None, backend="auto",
                                           deterministic=False, high_precision_level=0):
    validate_attention_scale(scale)
    return _call_bwd(sliding_window_softdelta_attention_bwd, "window", locals())


def sliding_chunk_softdelta_attention(q, k, k_read, v, g, chunk_size, scale=None, prev_k=None, prev_v=None,
                                      q_segment_idx=None, k_segment_idx=None, *, segment_idx=None,
                                      bos_mask=None, backend="auto", reset_chunk_pos_per_seq=False,
                                      deterministic=False, high_precision_level=0) -> Tensor:
    """SoftDelta over the query's chunk and the chunk before it; previous K/V, when given, holds
    exactly ``chunk_size`` tokens; ``reset_chunk_pos_per_seq`` restarts chunk positions per segment."""
    validate_attention_scale(scale)
    return _call(sliding_chunk_softdelta_attention, "chunk", locals())


@torch.no_grad()
def sliding_chunk_softdelta_attention_fwd(q, k, k_read, v, g, chunk_size, scale=None, prev_k=None,
                                          prev_v=None, q_segment_idx=None, k_segment_idx=None, *,
                                          segment_idx=None, bos_mask=None, backend="auto",
                                          reset_chunk_pos_per_seq=False, deterministic=False,
                                          high_precision_level=0):
    validate_attention_scale(scale)
    return _call_fwd(sliding_chunk_softdelta_attention_fwd, "chunk", locals())


@torch.no_grad()
def sliding_chunk_softdelta_attention_bwd(y_grad, q, k, k_read, v, g, y, neg_read, lse, chunk_size,
                                          scale=None, prev_k=None, prev_v=None, q_segment_idx=None,
                                          k_segment_idx=None, *, segment_idx=None, bos_mask=None,
                                          backend="auto", reset_chunk_pos_per_seq=False,
                                          deterministic=False, high_precision_level=0):
    """``(dq, dk, dv, dg, dk_read, dprev_k, dprev_v)``."""
    validate_attention_scale(scale)
    return _call_bwd(sliding_chunk_softdelta_attention_bwd, "chunk", locals())
