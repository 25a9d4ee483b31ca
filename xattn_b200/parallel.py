"""Sequence sharding of one long sequence across the GPUs of a node.

The reference is a single-GPU library; its chunk-to-chunk seam ``prev_k / prev_v -> dprev_k / dprev_v``
(docs/sliding_window_attention.md:31-37,78-79; xattn/ops/_causal_attention.py:170-198) is exactly what a
sequence-parallel run needs, and this module plugs communication into it:

* sliding-window and sliding-chunk attention: rank ``r`` holds a contiguous slice of the sequence and
  needs only the last ``window`` (or ``chunk``) keys / values of rank ``r-1`` — one send / recv of the
  K/V halo forward, one of ``dprev_k / dprev_v`` backward (added into rank ``r-1``'s dK / dV).
* causal attention: a ring.  At step ``t`` rank ``r`` reads the K/V block of rank ``r-t`` (diagonal
  block causal, earlier blocks unmasked, later blocks skipped), merges the partial outputs by their
  log-sum-exp, and prefetches the next block while computing.  The backward sends each block's dK / dV
  home.  With contiguous slices rank ``r`` has ``r + 1`` blocks of work; the ``zigzag`` layout (rank ``r``
  holds chunks ``r`` and ``2R-1-r`` of ``2R``) gives every rank the same work at every step: an earlier
  rank's block is seen by all local rows through its first chunk only, a later rank's block is seen
  whole by the local second chunk only, both unmasked.

Batch x heads sharding needs no code: ranks run independent batches.

Transport is ``torch.distributed`` point-to-point (NCCL over NVLink on GPUs, gloo in the CPU tests):
remote data always lands in a local buffer before a kernel reads it, so every TMA load is local.
The attention math is injected (``op`` / ``kernels`` arguments, defaulting to this package's CUDA
ops), which lets the CPU test-suite drive the communication logic with the oracle.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def _world(group) -> Tuple[int, int]:
    return dist.get_rank(group), dist.get_world_size(group)


def _global_rank(group, rank_in_group: int) -> int:
    return dist.get_global_rank(group, rank_in_group) if group is not None else rank_in_group


def _exchange(send: Optional[Tensor], send_to: Optional[int], recv: Optional[Tensor], recv_from: Optional[int],
              group) -> None:
    """One batched point-to-point step (either side may be absent at the ends of the chain)."""
    ops = []
    if send is not None and send_to is not None:
        ops.append(dist.P2POp(dist.isend, send.contiguous(), _global_rank(group, send_to), group))
    if recv is not None and recv_from is not None:
        ops.append(dist.P2POp(dist.irecv, recv, _global_rank(group, recv_from), group))
    if ops:
        for work in dist.batch_isend_irecv(ops):
            work.wait()


class _Halo(torch.autograd.Function):
    """(k, v) of this rank -> (k, v, prev_k, prev_v): the inputs passed through, plus the last
    ``halo`` tokens of the previous rank's K / V (zero-length on rank 0).

    Backward: the gradient of the received halo travels back to the previous rank and is added to the
    tail of its dK / dV.  K and V pass through the node so that every rank's graph contains it and
    takes part in that exchange, whether or not it used a halo itself."""

    @staticmethod
    def forward(ctx, k: Tensor, v: Tensor, halo: int, group):
        rank, world = _world(group)
        ctx.group, ctx.halo, ctx.rank, ctx.world = group, halo, rank, world
        n_prev = halo if rank > 0 else 0
        prev_k = k.new_empty((k.shape[0], n_prev, *k.shape[2:]))
        prev_v = v.new_empty((v.shape[0], n_prev, *v.shape[2:]))
        nxt = rank + 1 if rank + 1 < world else None
        prv = rank - 1 if rank > 0 else None
        _exchange(k[:, -halo:] if nxt is not None else None, nxt, prev_k if prv is not None else None, prv, group)
        _exchange(v[:, -halo:] if nxt is not None else None, nxt, prev_v if prv is not None else None, prv, group)
        return k.view_as(k), v.view_as(v), prev_k, prev_v

    @staticmethod
    def backward(ctx, dk: Optional[Tensor], dv: Optional[Tensor], dprev_k: Optional[Tensor], dprev_v: Optional[Tensor]):
        rank, world, halo, group = ctx.rank, ctx.world, ctx.halo, ctx.group
        nxt = rank + 1 if rank + 1 < world else None
        prv = rank - 1 if rank > 0 else None

        def step(grad_out, grad_halo):
            recv = grad_out.new_empty((grad_out.shape[0], halo, *grad_out.shape[2:])) if nxt is not None else None
            _exchange(grad_halo if prv is not None else None, prv, recv, nxt, group)
            if nxt is None:
                return grad_out
            total = grad_out.clone()
            total[:, -halo:] += recv
            return total

        return step(dk, dprev_k), step(dv, dprev_v), None, None


def _halo_ids(ids: Optional[Tensor], halo: int, group) -> Optional[Tensor]:
    """Segment ids of the halo tokens (no gradient): [previous rank's tail ‖ own ids]."""
    if ids is None:
        return None
    rank, world = _world(group)
    recv = ids.new_empty((ids.shape[0], halo)) if rank > 0 else None
    _exchange(ids[:, -halo:] if rank + 1 < world else None, rank + 1 if rank + 1 < world else None,
              recv, rank - 1 if rank > 0 else None, group)
    return ids if rank == 0 else torch.cat((recv, ids), dim=1)


def sequence_parallel_flash_swa(q: Tensor, k: Tensor, v: Tensor, window_size: int, scale: Optional[float] = None,
                                *, segment_idx: Optional[Tensor] = None, group=None,
                                op: Optional[Callable] = None, **op_kwargs) -> Tensor:
    """Sliding-window attention over a sequence split contiguously across the ranks of ``group``.

    ``q``, ``k``, ``v`` (and ``segment_idx`` ``[B, L_local]``, global ids) are this rank's slice; every
    rank's slice must hold at least ``window_size`` tokens so that the halo comes from one neighbour.
    Differentiable: dK / dV of the halo return to the rank that owns those tokens.
    """
    if op is None:
        from .ops import flash_swa as op
    if window_size <= 0:
        return op(q, k, v, window_size, scale, segment_idx=segment_idx, **op_kwargs)
    if k.shape[1] < window_size:
        raise ValueError("every rank's slice must be at least window_size tokens long")
    rank, _ = _world(group)
    k, v, prev_k, prev_v = _Halo.apply(k, v, window_size, group)
    ids = _halo_ids(segment_idx, window_size, group)
    if rank == 0:
        return op(q, k, v, window_size, scale, segment_idx=ids, **op_kwargs)
    return op(q, k, v, window_size, scale, prev_k, prev_v, segment_idx=ids, **op_kwargs)


def sequence_parallel_flash_sca(q: Tensor, k: Tensor, v: Tensor, chunk_size: int, scale: Optional[float] = None,
                                *, segment_idx: Optional[Tensor] = None, group=None,
                                op: Optional[Callable] = None, **op_kwargs) -> Tensor:
    """Sliding-chunk attention over a sequence split across ranks.  Slice lengths must be multiples of
    ``chunk_size`` so that global chunk boundaries survive the split; the halo is exactly one chunk
    (the reference's contract for previous K/V, xattn/ops/sliding_chunk_attention.py:538-541).
    Per-segment reset positions are not supported across ranks."""
    if op is None:
        from .ops import flash_sca as op
    if k.shape[1] % chunk_size:
        raise ValueError("every rank's slice must be a multiple of chunk_size long")
    if op_kwargs.get("reset_chunk_pos_per_seq"):
        raise ValueError("per-segment reset positions cannot be split across ranks")
    rank, _ = _world(group)
    k, v, prev_k, prev_v = _Halo.apply(k, v, chunk_size, group)
    ids = _halo_ids(segment_idx, chunk_size, group)
    if rank == 0:
        return op(q, k, v, chunk_size, scale, segment_idx=ids, **op_kwargs)
    return op(q, k, v, chunk_size, scale, prev_k, prev_v, segment_idx=ids, **op_kwargs)


# ---- causal ring ----------------------------------------------------------------------------------

class NativeBlockKernels:
    """Block-level forward / backward on this package's CUDA kernels."""

    @staticmethod
    def forward(q: Tensor, k: Tensor, v: Tensor, scale: float, causal: bool) -> Tuple[Tensor, Tensor]:
        """FP32 partial output [B, L, H, V] and its lse [B, H, L] for one K/V block."""
        from . import _native
        plan = _native.build_plan(q.shape[0], q.shape[1], k.shape[1], q.device, visibility="full" if causal else "all")
        state = torch.empty((*q.shape[:3], v.shape[3]), dtype=torch.float32, device=q.device)
        _, lse = _native.attention_fwd(q, k, v, plan, scale, output_state=state)
        return state, lse

    @staticmethod
    def backward(dy: Tensor, q: Tensor, k: Tensor, v: Tensor, y: Tensor, lse: Tensor, scale: float,
                 causal: bool) -> Tuple[Tensor, Tensor, Tensor]:
        """Gradients of one block given the merged output ``y`` and the global ``lse``."""
        from . import _native
        plan = _native.build_plan(q.shape[0], q.shape[1], k.shape[1], q.device, visibility="full" if causal else "all")
        return _native.attention_bwd(dy, q, k, v, y, lse, plan, scale)


def _merge(acc: Optional[Tuple[Tensor, Tensor]], y: Tensor, lse: Tensor) -> Tuple[Tensor, Tensor]:
    """Combine normalised partial outputs by their log-sum-exp (lse [B,H,L], y [B,L,H,V])."""
    wide = torch.float64 if y.dtype == torch.float64 else torch.float32
    y, lse = y.to(wide), lse.to(wide)
    if acc is None:
        return y, lse
    y0, l0 = acc
    new = torch.logaddexp(l0, lse)
    w0 = torch.exp(l0 - new).transpose(1, 2).unsqueeze(-1)
    w1 = torch.exp(lse - new).transpose(1, 2).unsqueeze(-1)
    w0 = torch.nan_to_num(w0, nan=0.0)   # both -inf: no visible key so far
    w1 = torch.nan_to_num(w1, nan=0.0)
    return y0 * w0 + y * w1, new


def zigzag_indices(length: int, rank: int, world: int) -> Tensor:
    """Positions of the full sequence that rank ``rank`` holds in the zig-zag layout: chunks ``rank`` and
    ``2 * world - 1 - rank`` of ``2 * world`` equal chunks, in order."""
    if length % (2 * world):
        raise ValueError("the zig-zag layout needs a sequence length that is a multiple of 2 * world size")
    c = length // (2 * world)
    return torch.cat((torch.arange(rank * c, (rank + 1) * c),
                      torch.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c)))


def _merge_rows(acc: Tuple[Tensor, Tensor], y: Tensor, lse: Tensor, start: int) -> Tuple[Tensor, Tensor]:
    """Merge a partial result that covers the rows from ``start`` on."""
    y0, l0 = acc
    ya, la = _merge((y0[:, start:], l0[:, :, start:]), y, lse)
    y0[:, start:] = ya
    l0[:, :, start:] = la
    return y0, l0


class _RingCausal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, scale: float, group, kernels, zigzag: bool = False):
        rank, world = _world(group)
        half = q.shape[1] // 2
        send_to, recv_from = (rank + 1) % world, (rank - 1) % world
        blk_k, blk_v = k.contiguous(), v.contiguous()
        acc = None
        for t in range(world):
            nxt_k = nxt_v = None
            pending = []
            if t + 1 < world:
                # prefetch the next block while this one is computed
                nxt_k, nxt_v = torch.empty_like(blk_k), torch.empty_like(blk_v)
                ops = [dist.P2POp(dist.isend, blk_k, _global_rank(group, send_to), group),
                       dist.P2POp(dist.irecv, nxt_k, _global_rank(group, recv_from), group),
                       dist.P2POp(dist.isend, blk_v, _global_rank(group, send_to), group),
                       dist.P2POp(dist.irecv, nxt_v, _global_rank(group, recv_from), group)]
                pending = dist.batch_isend_irecv(ops)
            if zigzag and t > 0:
                if t <= rank:   # an earlier rank's block: its first chunk lies before both local chunks
                    y_t, lse_t = kernels.forward(q, blk_k[:, :half], blk_v[:, :half], scale, causal=False)
                    acc = _merge(acc, y_t, lse_t)
                else:           # a later rank's block: both of its chunks lie between the local ones
                    y_t, lse_t = kernels.forward(q[:, half:], blk_k, blk_v, scale, causal=False)
                    acc = _merge_rows(acc, y_t, lse_t, half)
            elif t <= rank:     # the block of rank (rank - t): on or below the diagonal
                y_t, lse_t = kernels.forward(q, blk_k, blk_v, scale, causal=(t == 0))
                acc = _merge(acc, y_t, lse_t)
            for work in pending:
                work.wait()
            if t + 1 < world:
                blk_k, blk_v = nxt_k, nxt_v
        y32, lse = acc
        y = y32.to(q.dtype)
        ctx.save_for_backward(q, k, v, y, lse)
        ctx.scale, ctx.group, ctx.kernels, ctx.zigzag = scale, group, kernels, zigzag
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):
        q, k, v, y, lse = ctx.saved_tensors
        group, kernels, scale = ctx.group, ctx.kernels, ctx.scale
        rank, world = _world(group)
        zigzag, half = ctx.zigzag, q.shape[1] // 2
        send_to, recv_from = (rank + 1) % world, (rank - 1) % world
        dy = dy.contiguous()
        blk_k, blk_v = k.contiguous(), v.contiguous()
        # gradients of the block currently held travel around the ring with it and arrive home after
        # `world` steps
        wide = torch.float64 if q.dtype == torch.float64 else torch.float32
        dk_acc = torch.zeros(k.shape, dtype=wide, device=k.device)
        dv_acc = torch.zeros(v.shape, dtype=wide, device=v.device)
        dq = torch.zeros(q.shape, dtype=wide, device=q.device)
        for t in range(world):
            if zigzag and t > 0:
                if t <= rank:
                    dq_t, dk_t, dv_t = kernels.backward(dy, q, blk_k[:, :half], blk_v[:, :half], y, lse, scale,
                                                        causal=False)
                    dq += dq_t.to(wide)
                    dk_acc[:, :half] += dk_t.to(wide)
                    dv_acc[:, :half] += dv_t.to(wide)
                else:
                    dq_t, dk_t, dv_t = kernels.backward(dy[:, half:], q[:, half:], blk_k, blk_v, y[:, half:],
                                                        lse[:, :, half:], scale, causal=False)
                    dq[:, half:] += dq_t.to(wide)
                    dk_acc += dk_t.to(wide)
                    dv_acc += dv_t.to(wide)
            elif t <= rank:
                dq_t, dk_t, dv_t = kernels.backward(dy, q, blk_k, blk_v, y, lse, scale, causal=(t == 0))
                dq += dq_t.to(wide)
                dk_acc += dk_t.to(wide)
                dv_acc += dv_t.to(wide)
            # pass the block and its gradient accumulators on (the last step brings them home)
            bufs = [blk_k, blk_v, dk_acc, dv_acc]
            recv = [torch.empty_like(b) for b in bufs]
            ops = []
            for s_, r_ in zip(bufs, recv):
                ops.append(dist.P2POp(dist.isend, s_, _global_rank(group, send_to), group))
                ops.append(dist.P2POp(dist.irecv, r_, _global_rank(group, recv_from), group))
            for work in dist.batch_isend_irecv(ops):
                work.wait()
            blk_k, blk_v, dk_acc, dv_acc = recv
        return dq.to(q.dtype), dk_acc.to(k.dtype), dv_acc.to(v.dtype), None, None, None, None


def ring_causal_flash_attn(q: Tensor, k: Tensor, v: Tensor, scale: Optional[float] = None, *, group=None,
                           kernels=None, layout: str = "contiguous") -> Tensor:
    """Causal attention over a sequence split across ranks (equal slice lengths, no segment metadata):
    ring of K/V blocks, partial outputs merged by log-sum-exp, differentiable.

    ``layout="contiguous"``: rank r holds positions [r * n, (r + 1) * n).  ``layout="zigzag"``: rank r holds
    the positions ``zigzag_indices(length, r, world)`` (an even slice length), which balances the causal
    work: every rank computes half a block at every step."""
    if q.shape[1] != k.shape[1]:
        raise ValueError("ring attention needs equal query and key slice lengths")
    if layout not in ("contiguous", "zigzag"):
        raise ValueError("layout must be 'contiguous' or 'zigzag'")
    if layout == "zigzag" and q.shape[1] % 2:
        raise ValueError("the zig-zag layout needs an even slice length")
    s = float(scale) if scale is not None else q.shape[-1] ** -0.5
    return _RingCausal.apply(q, k, v, s, group, kernels or NativeBlockKernels, layout == "zigzag")
