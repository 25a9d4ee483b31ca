"""Sequence sharding (halo exchange for sliding windows / chunks, causal ring) on CPU ranks.

Two gloo processes drive xattn_b200.parallel with the attention math injected from the CPU oracle, and
compare the sharded result (outputs and every gradient, including the halo gradients that travel back
to the previous rank) with the oracle on the whole sequence."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ---- oracle-backed stand-ins for the CUDA ops ------------------------------------------------------

def _oracle_op(visibility):
    from oracle import attention_oracle as O

    def op(q, k, v, span, scale=None, prev_k=None, prev_v=None, *, segment_idx=None, **kw):
        q_ids = None if segment_idx is None else segment_idx[:, -q.shape[1]:]
        return O.attention(q, k, v, visibility=visibility, span=span, scale=scale, prev_k=prev_k, prev_v=prev_v,
                           q_segment_idx=q_ids, k_segment_idx=segment_idx)
    return op


class _OracleBlocks:
    """Block kernels for the ring, in FP64 torch: forward -> (normalised partial y, lse); backward from the
    merged y and the global lse (the formulas the CUDA backward implements)."""

    @staticmethod
    def _scores(q, k, scale, causal):
        g = q.shape[2] // k.shape[2]
        kk = k.repeat_interleave(g, 2) if g != 1 else k
        s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
        if causal:
            L = q.shape[1]
            mask = torch.ones(L, k.shape[1], dtype=torch.bool).tril(k.shape[1] - L)
            s = s.masked_fill(~mask, float("-inf"))
        return s, g

    @staticmethod
    def forward(q, k, v, scale, causal):
        s, g = _OracleBlocks._scores(q, k, scale, causal)
        lse = torch.logsumexp(s, -1)
        p = torch.exp(s - lse[..., None])
        vv = v.repeat_interleave(g, 2) if g != 1 else v
        return torch.einsum("bhqk,bkhv->bqhv", p, vv), lse

    @staticmethod
    def backward(dy, q, k, v, y, lse, scale, causal):
        s, g = _OracleBlocks._scores(q, k, scale, causal)
        p = torch.exp(s - lse[..., None])
        vv = v.repeat_interleave(g, 2) if g != 1 else v
        kk = k.repeat_interleave(g, 2) if g != 1 else k
        dp = torch.einsum("bqhv,bkhv->bhqk", dy, vv)
        delta = (dy * y).sum(-1).transpose(1, 2)
        ds = p * (dp - delta[..., None])
        dq = torch.einsum("bhqk,bkhd->bqhd", ds, kk) * scale
        dk = torch.einsum("bhqk,bqhd->bkhd", ds, q) * scale
        dv = torch.einsum("bhqk,bqhv->bkhv", p, dy)
        B, Lk, H, D = dk.shape
        dk = dk.view(B, Lk, H // g, g, D).sum(3)
        dv = dv.view(B, Lk, H // g, g, -1).sum(3)
        return dq, dk, dv


# ---- worker -------------------------------------------------------------------------------------------

def _worker(rank, world, port, mode, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attention_oracle as O
        from xattn_b200 import parallel as P
        if mode.endswith("+links"):
            # pair communicators for the neighbours; the exchanges must take them and give the same results
            mode = mode[:-len("+links")]
            P.open_neighbor_links()
            assert len(P._LINKS[None]) == (world if world > 2 else 0)
        uneven, twohop = mode == "swa-uneven", mode == "swa-twohop"
        if uneven or twohop:
            mode = "swa"
        torch.manual_seed(0)
        B, L, Hq, Hkv, D = 2, 48, 4, 2, 8
        q = torch.randn(B, L, Hq, D, dtype=torch.float64)
        k = torch.randn(B, L, Hkv, D, dtype=torch.float64)
        v = torch.randn(B, L, Hkv, D, dtype=torch.float64)
        dy = torch.randn(B, L, Hq, D, dtype=torch.float64)
        ids = (torch.arange(L) // 19).expand(B, -1).contiguous() if mode in ("swa", "sca") else None
        n = L // world
        sl = P.zigzag_indices(L, rank, world) if mode == "zigzag" else slice(rank * n, (rank + 1) * n)
        if uneven:
            # slices of different lengths (a caller balancing the work of a window workload): only the halo
            # has to have the same size on both sides of an exchange
            cuts = [0, 21, 34, L][:world] + [L]
            sl = slice(cuts[rank], cuts[rank + 1])
        lengths = None
        if twohop:
            # slices shorter than the window (13): ranks 2 and 3 take 10 rows from the previous rank and 3 from
            # the one before it, and the gradients go back the same two ways
            lengths = [18, 10, 10, 10]
            sl = slice(sum(lengths[:rank]), sum(lengths[:rank + 1]))
        ql, kl, vl = (t[:, sl].clone().requires_grad_() for t in (q, k, v))
        if mode == "swa":
            span = 13 if twohop else 7
            y = P.sequence_parallel_flash_swa(ql, kl, vl, span, segment_idx=ids[:, sl], op=_oracle_op("window"),
                                              slice_lengths=lengths)
            full = dict(visibility="window", span=span)
        elif mode == "sca":
            y = P.sequence_parallel_flash_sca(ql, kl, vl, 8, segment_idx=ids[:, sl], op=_oracle_op("chunk"))
            full = dict(visibility="chunk", span=8)
        else:
            y = P.ring_causal_flash_attn(ql, kl, vl, kernels=_OracleBlocks,
                                         layout="zigzag" if mode == "zigzag" else "contiguous",
                                         use_links=P.neighbor_links_open())
            full = dict(visibility="full")
        grads = torch.autograd.grad(y, (ql, kl, vl), dy[:, sl])
        ref_leaves = [t.clone().requires_grad_() for t in (q, k, v)]
        y_ref = O.attention(*ref_leaves, q_segment_idx=ids, k_segment_idx=ids, **full)
        g_ref = torch.autograd.grad(y_ref, ref_leaves, dy)
        errs = [(y - y_ref[:, sl]).abs().max().item()]
        errs += [(g - r[:, sl]).abs().max().item() for g, r in zip(grads, g_ref)]
        results[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ("swa", "sca", "ring", "zigzag"))
@pytest.mark.parametrize("world", (2, 3))
def test_sequence_sharding_matches_unsharded_oracle(mode, world):
    if mode == "sca" and world == 3:
        world = 2      # 48 / 3 = 16 is a multiple of 8 as well, but keep one 3-rank case per family short
    _run_ranks(mode, world)


@pytest.mark.parametrize("mode,world", (("swa-uneven", 3), ("swa-twohop", 4)))
def test_window_sharding_with_slices_of_different_lengths(mode, world):
    _run_ranks(mode, world)


@pytest.mark.parametrize("mode,world", (("swa+links", 3), ("ring+links", 3), ("zigzag+links", 4)))
def test_sequence_sharding_over_neighbor_links(mode, world):
    """The same results when every pair of neighbours talks over a communicator of its own."""
    _run_ranks(mode, world)


def _run_ranks(mode, world):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        # the rendezvous port is picked, released and then bound by rank 0: if another process takes it in
        # between, the ranks fail at start-up and the case is run once more on a new port
        for attempt in range(2):
            results = manager.dict()
            port = _free_port()
            procs = [ctx.Process(target=_worker, args=(r, world, port, mode, results)) for r in range(world)]
            for p in procs:
                p.start()
            for p in procs:
                p.join(timeout=300)
            for p in procs:
                if p.is_alive():
                    p.kill()
            if all(p.exitcode == 0 for p in procs) or attempt == 1:
                break
        for p in procs:
            assert p.exitcode == 0, f"rank exited with {p.exitcode}"
        assert len(results) == world
        assert max(results.values()) < 1e-10, dict(results)


# ---- the native autograd node, on CPU ------------------------------------------------------------------
# ``_ShardedLocalAttention`` (halo exchange + this package's kernels as one node, dK / dV before dQ) only runs
# on GPUs.  Its exchange logic is driven here with the two calls it makes into the CUDA layer replaced by
# the oracle: what is checked is which rows travel where and where the returned gradients are added.

def _native_node_worker(rank, world, port, lengths, span, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attention_oracle as O
        from xattn_b200 import _native, parallel as P
        from xattn_b200.ops import _core
        calls = {}

        def fake_forward(q, k_all, v_all, support, scale, prev_k, prev_v, q_ids, k_ids, *, return_plan=False, **kw):
            y = O.attention(q, k_all, v_all, visibility=support.kind, span=support.span, scale=scale,
                            q_segment_idx=q_ids, k_segment_idx=k_ids)
            plan = torch.zeros(1, dtype=torch.int32)
            calls[id(plan)] = (support, q_ids, k_ids)
            return y, torch.zeros(1), None, plan

        class FakeBackwardCall:
            def __init__(self, dy, q, k_all, v_all, y, lse, plan, scale):
                support, q_ids, k_ids = calls[id(plan)]
                with torch.enable_grad():          # an autograd backward runs with gradients off
                    leaves = [t.detach().clone().requires_grad_() for t in (q, k_all, v_all)]
                    out = O.attention(*leaves, visibility=support.kind, span=support.span, scale=scale,
                                      q_segment_idx=q_ids, k_segment_idx=k_ids)
                    self._grads = torch.autograd.grad(out, leaves, dy)
                self.dq = self.dk = self.dv = None
                self.phases = []

            def run(self, phases=0):
                self.phases.append(phases)
                if phases & 4:
                    self.dk, self.dv = self._grads[1].clone(), self._grads[2].clone()
                if phases & 2:
                    self.dq = self._grads[0].clone()

        _core.forward, _native.BackwardCall = fake_forward, FakeBackwardCall
        torch.manual_seed(0)
        B, L, Hq, Hkv, D = 1, sum(lengths), 4, 2, 8
        q = torch.randn(B, L, Hq, D, dtype=torch.float64)
        k = torch.randn(B, L, Hkv, D, dtype=torch.float64)
        v = torch.randn(B, L, Hkv, D, dtype=torch.float64)
        dy = torch.randn(B, L, Hq, D, dtype=torch.float64)
        ids = (torch.arange(L) // 19).expand(B, -1).contiguous()
        sl = slice(sum(lengths[:rank]), sum(lengths[:rank + 1]))
        ql, kl, vl = (t[:, sl].clone().requires_grad_() for t in (q, k, v))
        y = P._ShardedLocalAttention.apply(ql, kl, vl, "window", span, D ** -0.5, ids[:, sl], None, tuple(lengths))
        grads = torch.autograd.grad(y, (ql, kl, vl), dy[:, sl])
        ref_leaves = [t.clone().requires_grad_() for t in (q, k, v)]
        y_ref = O.attention(*ref_leaves, q_segment_idx=ids, k_segment_idx=ids, visibility="window", span=span)
        g_ref = torch.autograd.grad(y_ref, ref_leaves, dy)
        errs = [(y - y_ref[:, sl]).abs().max().item()]
        errs += [(g - r[:, sl]).abs().max().item() for g, r in zip(grads, g_ref)]
        results[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("lengths,span", (((24, 24), 7), ((21, 13, 14), 7), ((18, 10, 10, 10), 13)),
                         ids=("two-ranks", "uneven", "two-hop"))
def test_native_sharded_node_exchanges(lengths, span):
    world = len(lengths)
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        for attempt in range(2):
            results = manager.dict()
            port = _free_port()
            procs = [ctx.Process(target=_native_node_worker, args=(r, world, port, lengths, span, results))
                     for r in range(world)]
            for p in procs:
                p.start()
            for p in procs:
                p.join(timeout=300)
            for p in procs:
                if p.is_alive():
                    p.kill()
            if all(p.exitcode == 0 for p in procs) or attempt == 1:
                break
        for p in procs:
            assert p.exitcode == 0, f"rank exited with {p.exitcode}"
        assert len(results) == world
        assert max(results.values()) < 1e-10, dict(results)


def test_halo_routes():
    """Which ranks a halo comes from and goes to: the neighbours without slice lengths, as many preceding
    ranks as the halo needs with them (nearest first), nothing before rank 0."""
    from xattn_b200.parallel import _halo_routes
    assert _halo_routes(0, 4, 7, None) == ({}, {1: 7})
    assert _halo_routes(2, 4, 7, None) == ({1: 7}, {1: 7})
    assert _halo_routes(3, 4, 7, None) == ({1: 7}, {})
    lengths = [5888] + [3840] * 7
    assert _halo_routes(0, 8, 4096, lengths) == ({}, {1: 4096, 2: 256})
    assert _halo_routes(1, 8, 4096, lengths) == ({1: 4096}, {1: 3840, 2: 256})
    assert _halo_routes(4, 8, 4096, lengths) == ({1: 3840, 2: 256}, {1: 3840, 2: 256})
    assert _halo_routes(7, 8, 4096, lengths) == ({1: 3840, 2: 256}, {})
    # every row a rank receives is a row another rank sends
    for lengths, halo in (([18, 10, 10, 10], 13), ([3, 3, 3, 3, 30], 8), ([40, 2, 2], 5)):
        world = len(lengths)
        routes = [_halo_routes(r, world, halo, lengths) for r in range(world)]
        for r, (sources, _) in enumerate(routes):
            assert sum(sources.values()) == min(halo, sum(lengths[:r]))
            for hop, rows in sources.items():
                assert routes[r - hop][1][hop] == rows
        assert sum(sum(f.values()) for _, f in routes) == sum(sum(s_.values()) for s_, _ in routes)


def test_halo_requires_long_enough_slices():
    from xattn_b200 import parallel as P
    q = torch.zeros(1, 4, 1, 8)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        with pytest.raises(ValueError, match="window_size"):
            P.sequence_parallel_flash_swa(q, q, q, 9, op=_oracle_op("window"))
        with pytest.raises(ValueError, match="multiple of chunk_size"):
            P.sequence_parallel_flash_sca(q, q, q, 3, op=_oracle_op("chunk"))
    finally:
        dist.destroy_process_group()


def test_zigzag_indices_partition_the_sequence():
    from xattn_b200 import parallel as P
    for world in (1, 2, 3, 8):
        length = 16 * world
        parts = [P.zigzag_indices(length, r, world) for r in range(world)]
        assert all(p.numel() == length // world for p in parts)
        assert torch.equal(torch.cat(parts).sort().values, torch.arange(length))
        c = length // (2 * world)
        for r, p in enumerate(parts):
            # an early chunk and its mirror image: causal work per rank is the same
            assert p[0] == r * c and p[-1] == length - r * c - 1
            assert bool((p[1:] > p[:-1]).all())
    with pytest.raises(ValueError, match="multiple of 2"):
        P.zigzag_indices(10, 0, 2)
    q = torch.zeros(1, 3, 1, 8)
    with pytest.raises(ValueError, match="even slice"):
        P.ring_causal_flash_attn(q, q, q, layout="zigzag")
    with pytest.raises(ValueError, match="layout"):
        P.ring_causal_flash_attn(q, q, q, layout="striped")


def _failing_worker(rank, world, port, results):
    """Rank 1 leaves before the exchange (as a crashed rank would, between steps, with nothing in flight);
    rank 0 must come back from its halo exchange with an error instead of waiting for ever."""
    import datetime
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from xattn_b200 import parallel as P
    if rank == 1:
        results[rank] = "left"
        os._exit(0)                      # no destroy_process_group: the peer only sees the connection go
    q = torch.randn(1, 16, 2, 8, dtype=torch.float64)
    try:
        P.sequence_parallel_flash_swa(q, q[:, :, :1], q[:, :, :1], 4, op=_oracle_op("window"))
        results[rank] = "returned"
    except Exception as exc:             # gloo reports the closed connection or the timeout
        results[rank] = "error: " + type(exc).__name__


def test_a_rank_that_left_ends_the_halo_exchange_with_an_error():
    """Failure detection on the host side: no GPU is involved, nothing hangs.  The surviving rank's send to
    the rank that left fails (connection closed, or the process group's timeout), it reports the error and
    exits; a rank that is still alive after the grace period is killed."""
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=60)
        stragglers = [p for p in procs if p.is_alive()]
        for p in stragglers:
            p.kill()
            p.join()
        assert not stragglers, "the surviving rank did not return from the exchange"
        assert results.get(1) == "left"
        assert str(results.get(0, "")).startswith("error"), dict(results)
