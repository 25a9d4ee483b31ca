"""Sequence sharding of one long sequence across the GPUs of a node.

The reference is a single-GPU library; its chunk-to-chunk seam ``prev_k / prev_v -> dprev_k / dprev_v``
(docs/sliding_window_attention.md:31-37,78-79; xattn/ops/_causal_attention.py:170-198) is exactly what a
sequence-parallel run needs, and this module plugs communication into it:

* sliding-window and sliding-chunk attention: rank ``r`` holds a contiguous slice of the sequence and
  needs only the last ``window`` (or ``chunk``) keys / values of rank ``r-1`` — one batched send / recv of
  the K/V halo (and its segment ids) forward, landing in front of the rank's own K / V in one buffer,
  and one of the halo's dK / dV backward (added into rank ``r-1``'s dK / dV).
* causal attention: a ring.  At step ``t`` rank ``r`` reads the K/V block of rank ``r-t`` (diagonal
  block causal, earlier blocks unmasked, later blocks skipped), merges the partial outputs by their
  log-sum-exp, and prefetches the next block while computing.  In the backward each block's dK / dV
  accumulator travels with it and arrives home after a full turn; both the next block and the
  accumulator move while the kernels of a step run.  With contiguous slices rank ``r`` has ``r + 1`` blocks of work; the ``zigzag`` layout (rank ``r``
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

from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def _world(group) -> Tuple[int, int]:
    return dist.get_rank(group), dist.get_world_size(group)


def _global_rank(group, rank_in_group: int) -> int:
    return dist.get_global_rank(group, rank_in_group) if group is not None else rank_in_group


# Pair communicators of neighbouring ranks, by the group they were opened for (None = the default group).
_LINKS: dict = {}


def _links_key(group):
    return None if group is None or group is dist.group.WORLD else group


def open_neighbor_links(group=None, high_priority: bool = True) -> None:
    """Give every pair of neighbouring ranks of ``group`` (the ring's wrap-around pair included) a
    communicator of its own, which the exchanges of this module then use instead of ``group``'s.

    Why: inside an N-rank NCCL communicator a point-to-point transfer gets a share of the channels that
    shrinks with N (the 17 MB halo of the window benchmark took 83 us between 2 ranks and 240 us among 8,
    same data, same NVLink); a two-rank communicator keeps the two-rank figure at every N.
    ``high_priority`` puts the links' NCCL kernels on high-priority streams, so that a transfer posted
    while an attention kernel fills the GPU starts when the first of its CTAs retires, not after the last
    one was scheduled.

    Like ``torch.distributed.new_group`` this is a collective over the DEFAULT process group: every rank
    of the job calls it, with the same arguments, before the first sharded call.  Without it everything
    works on ``group``'s own communicator.  Two-rank groups need no links."""
    ranks = dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)
    world = len(ranks)
    links = {}
    if world > 2:
        options = None
        if high_priority and dist.get_backend(group) == "nccl":
            options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        # one fixed order for all ranks (new_group is collective and blocks)
        me = dist.get_rank()
        for a in range(world):
            b = (a + 1) % world
            link = dist.new_group(sorted((ranks[a], ranks[b])), pg_options=options)
            links[frozenset((a, b))] = link
            # A communicator is set up at its first use, by both of its ranks together.  Left to the first
            # exchange, a ring would deadlock there: every rank would set up the link to its successor first
            # and wait for a successor that is busy with its own.  So each link is used once here, in the one
            # order all ranks share.
            if me in (ranks[a], ranks[b]):
                probe = torch.zeros(1, device="cuda" if dist.get_backend(link) == "nccl" else "cpu")
                dist.all_reduce(probe, group=link)
    _LINKS[_links_key(group)] = links


def neighbor_links_open(group=None) -> bool:
    return _links_key(group) in _LINKS


def close_neighbor_links(group=None) -> None:
    """Forget the links of ``group`` (their communicators end with the process group teardown)."""
    _LINKS.pop(_links_key(group), None)


def _p2p(sends, send_to: Optional[int], recvs, recv_from: Optional[int], group, use_links: bool = True):
    """One batched point-to-point step: every tensor of ``sends`` goes to ``send_to``, every buffer of
    ``recvs`` is filled from ``recv_from`` (either side may be absent at the ends of the chain).  Returns
    the pending work handles; the caller waits when it needs the data, so whatever it launches in
    between runs beside the transfer.  Peers issue their sends and receives in the same order.  With
    neighbour links open (``open_neighbor_links``) the sends and the receives go out as one batch each on
    the communicator of their pair (``use_links=False`` keeps a step on ``group``'s own)."""
    rank = dist.get_rank(group)
    links = (_LINKS.get(_links_key(group)) or {}) if use_links else {}
    out_link = links.get(frozenset((rank, send_to))) if send_to is not None else None
    in_link = links.get(frozenset((rank, recv_from))) if recv_from is not None else None
    send_ops, recv_ops = [], []
    if send_to is not None:
        peer = _global_rank(group, send_to)
        send_ops = [dist.P2POp(dist.isend, t.contiguous(), peer, group if out_link is None else out_link) for t in sends]
    if recv_from is not None:
        peer = _global_rank(group, recv_from)
        recv_ops = [dist.P2POp(dist.irecv, t, peer, group if in_link is None else in_link) for t in recvs]
    if (out_link is None and in_link is None) or out_link is in_link:
        ops = send_ops + recv_ops
        return dist.batch_isend_irecv(ops) if ops else []
    works = []
    for ops in (send_ops, recv_ops):
        if ops:
            works += dist.batch_isend_irecv(ops)
    return works


def _wait(works) -> None:
    for work in works:
        work.wait()


def _halo_routes(rank: int, world: int, halo: int, lengths: Optional[Sequence[int]]):
    """Where this rank's halo comes from and which ranks it feeds.  Returns two dictionaries
    ``hop -> rows``: rows received from rank ``rank - hop`` and rows sent to rank ``rank + hop``.
    Without ``lengths`` (every slice holds at least ``halo`` tokens) that is the previous rank and the
    next one.  With the slice lengths of all ranks a slice may be shorter than the halo, which then
    reaches back over as many ranks as it takes (nearest first)."""
    def sources_of(r: int):
        out, need = {}, halo
        for s in range(r - 1, -1, -1):
            take = need if lengths is None else min(need, int(lengths[s]))
            if take > 0:
                out[r - s] = take
            need -= take
            if need <= 0 or lengths is None:
                break
        return out
    sources = sources_of(rank)
    feeds = {}
    for d in range(rank + 1, world):
        rows = sources_of(d).get(d - rank)
        if rows:
            feeds[d - rank] = rows
        if lengths is None:
            break
    return sources, feeds


def _assemble_halo(ctx, k: Tensor, v: Tensor, halo: int, ids: Optional[Tensor], group, lengths=None):
    """[the ``halo`` tokens before this rank's slice ‖ own tokens] for K, V and the segment ids; what the
    backward needs to know about the exchange is left on ``ctx``."""
    rank, world = _world(group)
    sources, feeds = _halo_routes(rank, world, halo, lengths)
    n_prev = sum(sources.values())
    # rows of the farthest source first: offset of every source's rows in the assembled buffer
    offsets, off = {}, 0
    for hop in sorted(sources, reverse=True):
        offsets[hop] = off
        off += sources[hop]
    ctx.group, ctx.n_prev, ctx.sources, ctx.feeds, ctx.offsets = group, n_prev, sources, feeds, offsets
    tensors = [k, v] + ([ids] if ids is not None else [])
    out = [t.new_empty((t.shape[0], n_prev + t.shape[1], *t.shape[2:])) for t in tensors]
    # a slice along the token axis is one block of memory only for a batch of one: otherwise the
    # halo lands in buffers of its own first
    direct = k.shape[0] == 1
    landing, works = {}, []
    for hop in sorted(set(sources) | set(feeds)):           # the same order on every rank
        rows_in, rows_out = sources.get(hop), feeds.get(hop)
        if rows_in:
            lo = offsets[hop]
            landing[hop] = [o[:, lo:lo + rows_in] if direct else o.new_empty((o.shape[0], rows_in, *o.shape[2:]))
                            for o in out]
        works += _p2p([t[:, -rows_out:] for t in tensors] if rows_out else [], rank + hop if rows_out else None,
                      landing.get(hop, []), rank - hop if rows_in else None, group)
    for o, t in zip(out, tensors):
        o[:, n_prev:].copy_(t)
    _wait(works)
    if not direct:
        for hop, bufs in landing.items():
            lo = offsets[hop]
            for o, l in zip(out, bufs):
                o[:, lo:lo + sources[hop]].copy_(l)
    return out[0], out[1], (out[2] if ids is not None else None)


def _return_halo_gradients(ctx, grads):
    """Start the halo rows' gradients on their way back to the ranks that own those tokens and post the
    receives for the gradients of the rows this rank fed to others.  Returns (works, own, received):
    ``own`` are the views of this rank's own rows, ``received`` maps hop -> buffers to add to their tails."""
    rank = dist.get_rank(ctx.group)
    works, received = [], {}
    for hop in sorted(set(ctx.sources) | set(ctx.feeds)):
        rows_in, rows_out = ctx.sources.get(hop), ctx.feeds.get(hop)
        sends = []
        if rows_in:
            lo = ctx.offsets[hop]
            sends = [g[:, lo:lo + rows_in] for g in grads]
        if rows_out:
            received[hop] = [g.new_empty((g.shape[0], rows_out, *g.shape[2:])) for g in grads]
        works += _p2p(sends, rank - hop if rows_in else None, received.get(hop, []), rank + hop if rows_out else None,
                      ctx.group)
    return works, [g[:, ctx.n_prev:] for g in grads], received


def _add_returned_gradients(own, received) -> None:
    for bufs in received.values():
        for g, r in zip(own, bufs):
            g[:, -r.shape[1]:] += r          # the gradients are the calling function's alone: updated in place


class _HaloAssemble(torch.autograd.Function):
    """(k, v) of this rank -> (k_all, v_all, ids_all): the ``halo`` tokens before this rank's slice (K / V and
    segment ids of the previous rank, or ranks) in front of this rank's own, in one buffer each.  The
    attention op then sees a query slice that is shorter than its keys and right-aligned to them, which is
    the reference's own short-Q contract (tests/_reference.py:47-49): no previous-K/V arguments, no
    concatenation inside the op.  One batched exchange per neighbour carries K, V and ids; this rank's own
    K / V are copied into place while it is in flight.

    Backward: the gradient of the halo rows travels back to the ranks that own them and is added to the
    tail of their dK / dV (the reference's ``dprev_k / dprev_v`` seam, docs/sliding_window_attention.md:78-79).
    K and V pass through this node on every rank, so every rank takes part in that exchange whether
    or not it received a halo itself."""

    @staticmethod
    def forward(ctx, k: Tensor, v: Tensor, halo: int, ids: Optional[Tensor], group, lengths):
        k_all, v_all, ids_all = _assemble_halo(ctx, k, v, halo, ids, group, lengths)
        if ids_all is not None:
            ctx.mark_non_differentiable(ids_all)
        return k_all, v_all, ids_all

    @staticmethod
    def backward(ctx, dk_all: Tensor, dv_all: Tensor, _ids):
        works, own, received = _return_halo_gradients(ctx, [dk_all, dv_all])
        _wait(works)
        _add_returned_gradients(own, received)
        return own[0], own[1], None, None, None, None


class _ShardedLocalAttention(torch.autograd.Function):
    """The halo exchange and this package's kernels as one autograd node, so that the backward can order
    its kernels around the exchange: dK / dV first, the halo rows' gradients start their way back to the
    ranks that own them, the dQ kernel runs meanwhile, and only then does this rank wait for the gradients
    coming from the ranks it fed.  (With the exchange in a node of its own, ``_HaloAssemble``, it can only
    start after the whole attention backward.)  Level 0, the library's own ops; everything else takes the
    generic path."""

    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, kind: str, span: int, scale: float, ids: Optional[Tensor], group,
                lengths):
        from .ops import _core
        k_all, v_all, ids_all = _assemble_halo(ctx, k, v, span, ids, group, lengths)   # leaves the routes on ctx
        q_ids = None if ids_all is None else ids_all[:, ids_all.shape[1] - q.shape[1]:]
        support = _core.Support(kind, span)
        y, lse, _, plan = _core.forward(q, k_all, v_all, support, scale, None, None, q_ids, ids_all, return_plan=True)
        ctx.save_for_backward(q, k_all, v_all, y, lse, plan)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):
        from . import _lib, _native
        q, k_all, v_all, y, lse, plan = ctx.saved_tensors
        call = _native.BackwardCall(dy, q, k_all, v_all, y, lse, plan, ctx.scale)
        call.run(_lib.BWD_PHASE_PRE | _lib.BWD_PHASE_DKV)
        works, own, received = _return_halo_gradients(ctx, [call.dk, call.dv])
        call.run(_lib.BWD_PHASE_DQ)                     # beside the exchange
        _wait(works)
        _add_returned_gradients(own, received)
        return call.dq, own[0], own[1], None, None, None, None, None, None


def _sequence_parallel_local(op, q, k, v, span, scale, segment_idx, group, op_kwargs, kind, lengths=None):
    if lengths is not None:
        rank, world = _world(group)
        lengths = tuple(int(n) for n in lengths)
        if len(lengths) != world or min(lengths) <= 0 or lengths[rank] != k.shape[1]:
            raise ValueError("slice_lengths must give the positive slice length of every rank, this rank's included")
    if op is None and not op_kwargs and q.is_cuda:
        s = float(scale) if scale is not None else q.shape[-1] ** -0.5
        return _ShardedLocalAttention.apply(q, k, v, kind, span, s, segment_idx, group, lengths)
    if op is None:
        from . import ops
        op = ops.flash_swa if kind == "window" else ops.flash_sca
    k_all, v_all, ids_all = _HaloAssemble.apply(k, v, span, segment_idx, group, lengths)
    return op(q, k_all, v_all, span, scale, segment_idx=ids_all, **op_kwargs)


def sequence_parallel_flash_swa(q: Tensor, k: Tensor, v: Tensor, window_size: int, scale: Optional[float] = None,
                                *, segment_idx: Optional[Tensor] = None, group=None,
                                op: Optional[Callable] = None, slice_lengths: Optional[Sequence[int]] = None,
                                **op_kwargs) -> Tensor:
    """Sliding-window attention over a sequence split contiguously across the ranks of ``group``.

    ``q``, ``k``, ``v`` (and ``segment_idx`` ``[B, L_local]``, global ids) are this rank's slice.  The slices
    need not be equally long (the first ``window_size`` rows of a sequence see fewer keys, so equal work
    means a longer first slice).  Without ``slice_lengths`` every rank's slice must hold at least
    ``window_size`` tokens, so that the halo comes from one neighbour; with the slice lengths of all ranks
    (the same list on every rank) a slice may be shorter and the halo is collected from as many preceding
    ranks as it takes.  Differentiable: dK / dV of the halo return to the ranks that own those tokens.
    """
    if window_size <= 0:
        if op is None:
            from .ops import flash_swa as op
        return op(q, k, v, window_size, scale, segment_idx=segment_idx, **op_kwargs)
    if slice_lengths is None and k.shape[1] < window_size:
        raise ValueError("every rank's slice must be at least window_size tokens long (or pass slice_lengths)")
    return _sequence_parallel_local(op, q, k, v, window_size, scale, segment_idx, group, op_kwargs, "window",
                                    slice_lengths)


def sequence_parallel_flash_sca(q: Tensor, k: Tensor, v: Tensor, chunk_size: int, scale: Optional[float] = None,
                                *, segment_idx: Optional[Tensor] = None, group=None,
                                op: Optional[Callable] = None, **op_kwargs) -> Tensor:
    """Sliding-chunk attention over a sequence split across ranks.  Slice lengths must be multiples of
    ``chunk_size`` so that global chunk boundaries survive the split (the halo, exactly one chunk, then
    shifts every local key position by a multiple of the chunk size).  Per-segment reset positions are
    not supported across ranks."""
    if k.shape[1] % chunk_size:
        raise ValueError("every rank's slice must be a multiple of chunk_size long")
    if op_kwargs.get("reset_chunk_pos_per_seq"):
        raise ValueError("per-segment reset positions cannot be split across ranks")
    return _sequence_parallel_local(op, q, k, v, chunk_size, scale, segment_idx, group, op_kwargs, "chunk")


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

    @staticmethod
    def merge(acc: Tuple[Tensor, Tensor], y: Tensor, lse: Tensor, start: int = 0) -> Tuple[Tensor, Tensor]:
        """Fold a block's partial result into the running one, in place, with one kernel."""
        from . import _native
        _native.merge_partial_outputs(acc[0], acc[1], y, lse, start)
        return acc


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
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, scale: float, group, kernels, zigzag: bool = False,
                use_links: bool = False):
        rank, world = _world(group)
        half = q.shape[1] // 2
        send_to, recv_from = (rank + 1) % world, (rank - 1) % world
        blk_k, blk_v = k.contiguous(), v.contiguous()
        acc = None
        native_merge = getattr(kernels, "merge", None)

        def fold(acc, y_t, lse_t, start):
            """Running result after one more block; the block kernels' own merge where they have one."""
            if acc is None:
                return _merge(None, y_t, lse_t)
            if native_merge is not None:
                return native_merge(acc, y_t, lse_t, start)
            return _merge_rows(acc, y_t, lse_t, start) if start else _merge(acc, y_t, lse_t)

        for t in range(world):
            nxt_k = nxt_v = None
            pending = []
            if t + 1 < world:
                # prefetch the next block while this one is computed
                nxt_k, nxt_v = torch.empty_like(blk_k), torch.empty_like(blk_v)
                pending = _p2p([blk_k, blk_v], send_to, [nxt_k, nxt_v], recv_from, group, use_links)
            if zigzag and t > 0:
                if t <= rank:   # an earlier rank's block: its first chunk lies before both local chunks
                    y_t, lse_t = kernels.forward(q, blk_k[:, :half], blk_v[:, :half], scale, causal=False)
                    acc = fold(acc, y_t, lse_t, 0)
                else:           # a later rank's block: both of its chunks lie between the local ones
                    y_t, lse_t = kernels.forward(q[:, half:], blk_k, blk_v, scale, causal=False)
                    acc = fold(acc, y_t, lse_t, half)
            elif t <= rank:     # the block of rank (rank - t): on or below the diagonal
                y_t, lse_t = kernels.forward(q, blk_k, blk_v, scale, causal=(t == 0))
                acc = fold(acc, y_t, lse_t, 0)
            _wait(pending)
            if t + 1 < world:
                blk_k, blk_v = nxt_k, nxt_v
        y32, lse = acc
        y = y32.to(q.dtype)
        ctx.save_for_backward(q, k, v, y, lse)
        ctx.scale, ctx.group, ctx.kernels, ctx.zigzag, ctx.use_links = scale, group, kernels, zigzag, use_links
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
        # The K/V block held at step t came from rank - t; its dK / dV accumulate as it travels and are
        # home after `world` steps.  Two transfers per step, both beside the kernels: the NEXT block's K / V
        # (they never change, so they are requested before this step's kernels start), and the gradient
        # accumulator of the block just worked on, which the previous rank sent on after ITS step and which
        # is only needed once this step's own contribution exists.
        wide = torch.float64 if q.dtype == torch.float64 else torch.float32
        dq = torch.zeros(q.shape, dtype=wide, device=q.device)
        acc_in = None          # (works, dk, dv): the accumulator of the current block, arriving
        sent = []              # keep buffers of sends in flight alive until their work is done
        for t in range(world):
            nxt_k = nxt_v = None
            kv_works = []
            if t + 1 < world:
                nxt_k, nxt_v = torch.empty_like(blk_k), torch.empty_like(blk_v)
                kv_works = _p2p([blk_k, blk_v], send_to, [nxt_k, nxt_v], recv_from, group, ctx.use_links)
            dk_t = dv_t = None
            rows = slice(None)
            if zigzag and t > 0:
                if t <= rank:
                    dq_t, dk_t, dv_t = kernels.backward(dy, q, blk_k[:, :half], blk_v[:, :half], y, lse, scale,
                                                        causal=False)
                    dq += dq_t
                    rows = slice(0, half)
                else:
                    dq_t, dk_t, dv_t = kernels.backward(dy[:, half:], q[:, half:], blk_k, blk_v, y[:, half:],
                                                        lse[:, :, half:], scale, causal=False)
                    dq[:, half:] += dq_t
            elif t <= rank:
                dq_t, dk_t, dv_t = kernels.backward(dy, q, blk_k, blk_v, y, lse, scale, causal=(t == 0))
                dq += dq_t
            # this block's accumulator: zero on its home rank (t == 0), else what the previous rank sent on
            if acc_in is None:
                dk_acc = torch.zeros(k.shape, dtype=wide, device=k.device)
                dv_acc = torch.zeros(v.shape, dtype=wide, device=v.device)
            else:
                _wait(acc_in[0])
                dk_acc, dv_acc = acc_in[1], acc_in[2]
            if dk_t is not None:
                dk_acc[:, rows] += dk_t          # FP32 accumulators take the 16-bit results as they are
                dv_acc[:, rows] += dv_t
            # pass the accumulator on (the last step brings it home) and ask for the next one
            recv_dk, recv_dv = torch.empty_like(dk_acc), torch.empty_like(dv_acc)
            works = _p2p([dk_acc, dv_acc], send_to, [recv_dk, recv_dv], recv_from, group, ctx.use_links)
            sent.append((dk_acc, dv_acc))
            acc_in = (works, recv_dk, recv_dv)
            _wait(kv_works)
            if t + 1 < world:
                blk_k, blk_v = nxt_k, nxt_v
        _wait(acc_in[0])
        dk_home, dv_home = acc_in[1], acc_in[2]
        return dq.to(q.dtype), dk_home.to(k.dtype), dv_home.to(v.dtype), None, None, None, None, None


def ring_causal_flash_attn(q: Tensor, k: Tensor, v: Tensor, scale: Optional[float] = None, *, group=None,
                           kernels=None, layout: str = "contiguous", use_links: bool = False) -> Tensor:
    """Causal attention over a sequence split across ranks (equal slice lengths, no segment metadata):
    ring of K/V blocks, partial outputs merged by log-sum-exp, differentiable.

    ``layout="contiguous"``: rank r holds positions [r * n, (r + 1) * n).  ``layout="zigzag"``: rank r holds
    the positions ``zigzag_indices(length, r, world)`` (an even slice length), which balances the causal
    work: every rank computes half a block at every step.

    ``use_links``: send the blocks over the neighbour links (``open_neighbor_links``) instead of ``group``'s own
    communicator.  Off by default: NCCL connects two ranks for point-to-point traffic at their first
    transfer, with both of them present, and in a ring every rank would be waiting for its successor at that
    moment.  Turn it on once the links have carried a chain exchange (a sharded window or chunk call), which
    connects the pairs one after the other; the wrap-around pair then connects at the ring's first step."""
    if q.shape[1] != k.shape[1]:
        raise ValueError("ring attention needs equal query and key slice lengths")
    if layout not in ("contiguous", "zigzag"):
        raise ValueError("layout must be 'contiguous' or 'zigzag'")
    if layout == "zigzag" and q.shape[1] % 2:
        raise ValueError("the zig-zag layout needs an even slice length")
    s = float(scale) if scale is not None else q.shape[-1] ** -0.5
    return _RingCausal.apply(q, k, v, s, group, kernels or NativeBlockKernels, layout == "zigzag", bool(use_links))
