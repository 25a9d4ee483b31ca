"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch on the CPU, the algorithm the reference
checks its kernels against.  Only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it; the
product path never does (it fails loudly when the CUDA library is missing).

What it follows in the reference (paths inside the ifm-ai/xattn tree):

* visibility of a (query, key) pair        tests/_reference.py:35-131
  (``_allowed_masks``: right alignment ``q_pos = i + Lk - Lq`` :47-49, window
  ``k >= q_pos - span`` :54, chunk ``k >= (q_pos // span) * span - span`` :57,
  per-segment reset positions :92-110, strict-past variant :60-63,126-127)
* masked softmax read in FP64              tests/_reference.py:134-155
  (``_attention_from_mask``: rows without a visible key produce zeros)
* SoftDelta composition                    tests/softdelta/reference.py:9-71
  (``y = read - sigmoid(g) * neg_read``; the negative read queries with
  ``k_read`` over the strict past)
* tolerances                               tests/_reference.py:7-20

Parity pin: ``tests/golden/`` holds outputs of those reference functions run in
the build container (generator script next to the fixtures);
``tests/test_oracle.py`` checks this restatement against them.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor

# tests/_reference.py:7-20
ATOL = {torch.float16: 2e-4, torch.bfloat16: 1e-3}
GRAD_ATOL = {torch.float16: 2e-4, torch.bfloat16: 2e-3}
RTOL = {torch.float16: 1e-3, torch.bfloat16: 1e-2}


def _run_bounds(ids: Tensor) -> Tuple[Tensor, Tensor]:
    """For int64 ids [B, L]: start and end (exclusive) of the maximal run of
    equal neighbours that contains each position."""
    batch, length = ids.shape
    pos = torch.arange(length).expand(batch, length)
    first = torch.ones_like(ids, dtype=torch.bool)
    last = torch.ones_like(ids, dtype=torch.bool)
    if length > 1:
        change = ids[:, 1:] != ids[:, :-1]
        first[:, 1:] = change
        last[:, :-1] = change
    start = torch.where(first, pos, torch.zeros_like(pos)).cummax(dim=1).values
    end_marks = torch.where(last, pos + 1, torch.full_like(pos, length))
    end = end_marks.flip(1).cummin(dim=1).values.flip(1)
    return start, end


def allowed_masks(
    q_length: int,
    k_length: int,
    batch: int,
    visibility: str,
    span: Optional[int],
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    reset_position_per_segment: bool = False,
    rows: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor]:
    """(inclusive, strict-past) boolean masks [B, Lq, Lk].

    Restates tests/_reference.py:35-131 with array operations in place of the
    per-element loops.  Per-segment reset positions need each id to label one
    contiguous run per row (the reference asserts that, :29).

    ``rows`` (1-D indices of query rows) restricts the result to those rows, [B, len(rows), Lk]: the
    same rule evaluated for a sample of a sequence too long for the full matrix (the reference's
    long-sequence checks sample rows the same way, tests/_numerics.py:293-320).
    """
    if visibility not in ("full", "window", "chunk"):
        raise AssertionError(visibility)
    pick = torch.arange(q_length) if rows is None else rows.long()
    n_rows = pick.numel()
    k_index = torch.arange(k_length).expand(batch, k_length)
    aligned_q_pos = (pick + (k_length - q_length)).expand(batch, n_rows)
    if q_segment_idx is None:
        same = torch.ones(batch, n_rows, k_length, dtype=torch.bool)
        q_pos = aligned_q_pos
        k_pos = k_index[:, None, :].expand(batch, n_rows, k_length)
    else:
        assert k_segment_idx is not None
        q_ids = q_segment_idx.detach().cpu().long()
        k_ids = k_segment_idx.detach().cpu().long()
        same = q_ids[:, pick, None] == k_ids[:, None, :]
        if reset_position_per_segment:
            q_start, q_end = _run_bounds(q_ids)
            k_start, _ = _run_bounds(k_ids)
            matching = same.sum(dim=-1)  # length of the key run with the query's id (0 if none)
            q_pos = (pick[None, :] - q_start[:, pick]) + matching - (q_end - q_start)[:, pick]
            k_local = torch.arange(k_length)[None, :] - k_start
            k_pos = k_local[:, None, :].expand(batch, n_rows, k_length)
        else:
            q_pos = aligned_q_pos
            k_pos = k_index[:, None, :].expand(batch, n_rows, k_length)
    qp = q_pos[:, :, None]
    if visibility == "full":
        left = torch.ones(batch, n_rows, k_length, dtype=torch.bool)
    elif visibility == "window":
        assert span is not None
        left = k_pos >= qp - span
    else:
        assert span is not None
        left = k_pos >= torch.div(qp, span, rounding_mode="floor") * span - span
    inclusive = same & left & (k_pos <= qp)
    strict = same & left & (k_pos < qp)
    return inclusive, strict


def attention_from_mask(q: Tensor, k: Tensor, v: Tensor, allowed: Tensor, scale: float) -> Tensor:
    """Masked softmax read, tests/_reference.py:134-155.  q [B,Lq,Hq,D], k [B,Lk,Hkv,D],
    v [B,Lk,Hkv,V], allowed [B,Lq,Lk] -> [B,Lq,Hq,V] in the dtype of the inputs."""
    batch, q_len, heads, _ = q.shape
    kv_heads = k.shape[2]
    group = heads // kv_heads
    # the query heads of a KV group share its keys and values (repeat_interleave in the reference;
    # grouped here so that long sequences do not materialise repeated K and V)
    qg = q.reshape(batch, q_len, kv_heads, group, q.shape[-1])
    scores = torch.einsum("bqhgd,bkhd->bhgqk", qg, k) * scale
    keep = allowed[:, None, None]
    scores = scores.masked_fill(~keep, float("-inf"))
    any_key = allowed.any(dim=-1, keepdim=True)[:, None, None]
    scores = torch.where(any_key, scores, torch.zeros_like(scores))
    prob = torch.softmax(scores, dim=-1).masked_fill(~keep, 0.0)
    out = torch.einsum("bhgqk,bkhv->bqhgv", prob, v)
    return out.reshape(batch, q_len, heads, v.shape[-1])


def lse_from_mask(q: Tensor, k: Tensor, allowed: Tensor, scale: float) -> Tensor:
    """Natural-log sum of exp(scale * q.k) over visible keys, [B,Hq,Lq]; -inf for empty rows."""
    group = q.shape[2] // k.shape[2]
    if group != 1:
        k = k.repeat_interleave(group, dim=2)
    scores = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    scores = scores.masked_fill(~allowed[:, None], float("-inf"))
    return torch.logsumexp(scores, dim=-1)


def attention(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    *,
    visibility: str = "full",
    span: Optional[int] = None,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    reset_position_per_segment: bool = False,
    strict_past: bool = False,
) -> Tensor:
    """Full oracle call: concatenates previous K/V (tests/_numerics.py:170-178), builds the mask, reads."""
    if prev_k is not None:
        k = torch.cat((prev_k, k), dim=1)
        v = torch.cat((prev_v, v), dim=1)
    inc, strict = allowed_masks(q.shape[1], k.shape[1], q.shape[0], visibility, span,
                                q_segment_idx, k_segment_idx, reset_position_per_segment)
    s = q.shape[-1] ** -0.5 if scale is None else float(scale)
    return attention_from_mask(q, k, v, strict if strict_past else inc, s)


def softdelta(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    g: Tensor,
    k_read: Optional[Tensor] = None,
    *,
    scale: Optional[float] = None,
    prev_k: Optional[Tensor] = None,
    prev_v: Optional[Tensor] = None,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    visibility: str = "full",
    span: Optional[int] = None,
    reset_position_per_segment: bool = False,
):
    """SoftDelta, tests/softdelta/reference.py:9-71.  Scalar gates (``v`` [B, L, Hkv, V], ``g`` [B, Lq, H])
    or value groups (``v`` [B, L, Hkv, C, Dg], ``g`` [B, Lq, H, C, 1]: one gate per group of Dg channels,
    :36-71); the outputs follow the input layout.  Returns (y, read, neg_read)."""
    scalar = v.dim() == 4
    if scalar:
        v, g = v.unsqueeze(3), g[..., None, None]
        prev_v = None if prev_v is None else prev_v.unsqueeze(3)
    batch, length, q_heads, _ = q.shape
    if k_read is None:
        k_read = k[:, k.shape[1] - length:]
    if prev_k is not None:
        k = torch.cat((prev_k, k), dim=1)
        v = torch.cat((prev_v, v), dim=1)
    kv_heads = k.shape[2]
    groups, group_dim = v.shape[3:]
    s = q.shape[-1] ** -0.5 if scale is None else float(scale)
    inc, strict = allowed_masks(length, k.shape[1], batch, visibility, span,
                                q_segment_idx, k_segment_idx, reset_position_per_segment)
    flat_v = v.flatten(3)
    read = attention_from_mask(q, k, flat_v, inc, s)
    neg = attention_from_mask(k_read, k, flat_v, strict, s)
    rep = q_heads // kv_heads
    read = read.reshape(batch, length, kv_heads, rep, groups, group_dim)
    neg = neg.reshape(batch, length, kv_heads, 1, groups, group_dim)
    gate = torch.sigmoid(g).reshape(batch, length, kv_heads, rep, groups, 1)
    y = (read - gate * neg).reshape(batch, length, q_heads, groups, group_dim)
    read = read.reshape(batch, length, q_heads, groups, group_dim)
    neg = neg.reshape(batch, length, kv_heads, groups, group_dim)
    if scalar:
        y, read, neg = y.flatten(3), read.flatten(3), neg.flatten(3)
    return y, read, neg


def row_intervals(
    q_length: int,
    k_length: int,
    batch: int,
    visibility: str,
    span: Optional[int],
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
    reset_position_per_segment: bool = False,
    strict_past: bool = False,
) -> Tuple[Tensor, Tensor]:
    """Visible keys of each query row as a half-open interval [lo, hi) — what
    the device pre-pass produces.  Derived from ``allowed_masks`` (first/last
    visible key); also asserts that the visible set really is one interval."""
    inc, strict = allowed_masks(q_length, k_length, batch, visibility, span,
                                q_segment_idx, k_segment_idx, reset_position_per_segment)
    mask = strict if strict_past else inc
    count = mask.sum(-1)
    idx = torch.arange(k_length).expand_as(mask)
    lo = torch.where(mask, idx, torch.full_like(idx, k_length)).amin(-1) if k_length else count
    hi = torch.where(mask, idx + 1, torch.zeros_like(idx)).amax(-1) if k_length else count
    empty = count == 0
    lo = torch.where(empty, torch.zeros_like(lo), lo)
    hi = torch.where(empty, torch.zeros_like(hi), hi)
    assert bool(((hi - lo) == count).all()), "visible keys of a row are not one interval"
    return lo.to(torch.int32), hi.to(torch.int32)


def visible_pairs(lo: Tensor, hi: Tensor) -> int:
    """Number of visible (query, key) pairs of one head, for FLOP accounting."""
    return int((hi.long() - lo.long()).clamp_min(0).sum())


def forward_backward(q, k, v, dy, *, scale=None, **mask_kwargs):
    """FP-typed fwd + autograd bwd of ``attention`` (used for the timed CPU baseline)."""
    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    prev = {}
    for name in ("prev_k", "prev_v"):
        if mask_kwargs.get(name) is not None:
            prev[name] = mask_kwargs[name].detach().clone().requires_grad_()
            mask_kwargs[name] = prev[name]
    y = attention(*leaves, scale=scale, **mask_kwargs)
    grads = torch.autograd.grad(y, leaves + list(prev.values()), dy)
    return y.detach(), grads


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
