"""Edge sizes and regressions the reference pins in its own suite: very large batches
(tests/test_large_batch.py:16-112), long sequences checked on sampled rows with sparse dO
(tests/_numerics.py:293-320), the rounding-bias regression with identical keys (:216-235), and
live previous-K/V gradients under BOS masks (tests/test_high_precision.py:166-190)."""
import pytest
import torch
import torch.nn.functional as F

import xattn_b200 as xattn
from oracle import attention_oracle as O
from tests._cases import Case, make_inputs, metadata_for, op_options

pytestmark = pytest.mark.gpu
OPS = {"full": "causal_flash_attn", "window": "flash_swa", "chunk": "flash_sca"}


def test_large_batch_equals_chunked_batches(cuda_device):
    """More batch rows than a grid dimension holds: the result equals the same rows run in pieces."""
    dev = cuda_device
    torch.manual_seed(0)
    B, L, Hq, Hkv, D = 66000, 8, 2, 1, 32
    q = torch.randn(B, L, Hq, D, device=dev, dtype=torch.bfloat16)
    k = torch.randn(B, L, Hkv, D, device=dev, dtype=torch.bfloat16)
    v = torch.randn(B, L, Hkv, D, device=dev, dtype=torch.bfloat16)
    y, lse = xattn.causal_flash_attn_fwd(q, k, v)
    dy = torch.randn_like(y)
    grads = xattn.causal_flash_attn_bwd(dy, q, k, v, y, lse)
    for lo in (0, 40000):
        hi = min(lo + 40000, B)
        ys, ls = xattn.causal_flash_attn_fwd(q[lo:hi], k[lo:hi], v[lo:hi])
        assert torch.equal(ys, y[lo:hi]) and torch.equal(ls, lse[lo:hi])
        gs = xattn.causal_flash_attn_bwd(dy[lo:hi], q[lo:hi], k[lo:hi], v[lo:hi], ys, ls)
        for a, b in zip(gs, grads):
            assert torch.equal(a, b[lo:hi])
    ref = O.attention(q[:64].double().cpu(), k[:64].double().cpu(), v[:64].double().cpu())
    torch.testing.assert_close(y[:64].cpu().double(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("operation", OPS)
@pytest.mark.parametrize("length", (4096, 65536, 102400))
def test_long_sequences_on_sampled_rows(operation, length, cuda_device):
    """Sampled query rows against all keys; the gradient of those rows alone (sparse dO) is checked on
    the full-sized dq, dk, dv.  At 102400 a key tile is seen by 800 query tiles, more than the dK / dV
    kernel keeps tile bits for in shared memory (768): the last sampled rows go through its fallback."""
    dev = cuda_device
    dtype = torch.bfloat16
    span = 255
    gen = torch.Generator().manual_seed(length)
    H, Hkv, D = 4, 2, 64
    q = F.normalize(torch.randn(1, length, H, D, generator=gen), dim=-1).to(dev, dtype).requires_grad_()
    k = F.normalize(torch.randn(1, length, Hkv, D, generator=gen), dim=-1).to(dev, dtype).requires_grad_()
    v = (F.silu(torch.randn(1, length, Hkv, D, generator=gen)) + 0.1).to(dev, dtype).requires_grad_()
    rows = torch.tensor(sorted({0, 1, 127, 128, 191, 192, 255, 256, 257, 511, 512, length // 2, length - 2, length - 1}))
    kw = {"window": dict(window_size=span), "chunk": dict(chunk_size=span)}.get(operation, {})
    y = getattr(xattn, OPS[operation])(q, k, v, **kw)
    assert torch.isfinite(y).all()
    sel = y[:, rows.to(dev)]
    refs = [t.detach().double().cpu().requires_grad_() for t in (q, k, v)]
    qp = rows[:, None]
    kp = torch.arange(length)[None, :]
    left = torch.ones_like(kp, dtype=torch.bool).expand(len(rows), -1)
    if operation == "window":
        left = kp >= qp - span
    elif operation == "chunk":
        left = kp >= qp // span * span - span
    mask = (left & (kp <= qp))[None]
    expected = O.attention_from_mask(refs[0][:, rows], refs[1], refs[2], mask, D ** -0.5)
    torch.testing.assert_close(sel.detach().cpu(), expected.detach().to(dtype), atol=O.ATOL[dtype], rtol=O.RTOL[dtype])
    dy = (torch.randn(sel.shape, generator=gen) / sel.numel() ** 0.5).to(dev, dtype)
    grads = torch.autograd.grad(sel, (q, k, v), dy)
    want = torch.autograd.grad(expected, refs, dy.double().cpu())
    for g_, w_ in zip(grads, want):
        torch.testing.assert_close(g_.cpu(), w_.to(dtype), atol=O.GRAD_ATOL[dtype], rtol=O.RTOL[dtype])


@pytest.mark.parametrize("operation", ("window", "chunk"))
def test_rounding_bias_identical_keys(operation, cuda_device):
    """Identical key rows make dQ exactly zero whatever V and Q are; level 1 must not accumulate a bias."""
    dev = cuda_device
    q = torch.zeros(1, 128, 1, 64, dtype=torch.bfloat16, device=dev, requires_grad=True)
    k = torch.ones_like(q, requires_grad=True)
    values = torch.full_like(q, -1.0078125)
    values[:, :32] = -1.0
    fn = getattr(xattn, OPS[operation])
    options = {"chunk_size": 64} if operation == "chunk" else {"window_size": 127}
    dy = torch.zeros_like(q)
    dy[:, -1] = -1
    total = torch.zeros_like(q, dtype=torch.float64)
    for step in range(4):
        v = values.roll(step, 1).detach().requires_grad_()
        y = fn(q, k, v, **options, high_precision_level=1)
        dq = torch.autograd.grad(y, q, dy)[0]
        assert y.dtype == torch.bfloat16 and dq.abs().max() <= 1e-4
        total += dq.double()
    assert total.abs().max() <= 1e-3


@pytest.mark.parametrize("operation,reset", (("window", False), ("chunk", False), ("chunk", True)))
@pytest.mark.parametrize("level", (0, 1))
@pytest.mark.parametrize("kv_heads", (1, 2, 4))
def test_live_bos_previous_gradients(operation, reset, level, kv_heads, cuda_device):
    """Previous K/V that the current queries really read receive gradients of the right size."""
    dtype = torch.bfloat16
    case = Case("live-bos-previous", 129, 129, 128, 96, metadata="bos", previous=64, span=64, reset=reset, batch=1)
    inputs = make_inputs(operation, case, dtype, kv_heads, cuda_device)
    meta, qi, ki = metadata_for(case, cuda_device)
    options = {**op_options(operation, case, inputs), **meta}
    y = getattr(xattn, OPS[operation])(*inputs[:3], **options, high_precision_level=level)
    dy = torch.randn_like(y)
    grads = torch.autograd.grad(y, inputs, dy)
    refs = [t.detach().double().cpu().requires_grad_() for t in inputs]
    kk, vv = torch.cat((refs[3], refs[1]), 1), torch.cat((refs[4], refs[2]), 1)
    inc, _ = O.allowed_masks(129, 193, 1, operation, 64, qi.cpu(), ki.cpu(), reset)
    expected = O.attention_from_mask(refs[0], kk, vv, inc, 128 ** -0.5)
    want = torch.autograd.grad(expected, refs, dy.double().cpu())
    for g_, w_ in zip(grads[-2:], want[-2:]):
        assert w_.norm() > 0, "fixture must exercise live previous K/V"
        assert g_.dtype == dtype and g_.shape == w_.shape and torch.isfinite(g_).all()
        assert (g_.double().cpu() - w_).norm() <= 0.02 * w_.norm() + 1e-6


@pytest.mark.parametrize("operation", OPS)
@pytest.mark.parametrize("dims", ((40, 72), (136, 120), (152, 152), (56, 248)))
@pytest.mark.parametrize("level", (0, 1))
def test_padded_gqa_gradients(operation, dims, level, cuda_device):
    """Head dimensions that are not tile multiples, short Q, unit-variance dO: relative norm error of
    every gradient below 1.5 % (tests/test_high_precision.py:143-164)."""
    dtype = torch.bfloat16
    case = Case("padded-gqa", 17, 33, *dims, span=16, batch=1)
    inputs = make_inputs(operation, case, dtype, 2, cuda_device)
    options = op_options(operation, case, inputs)
    name = OPS[operation]
    y, lse = getattr(xattn, name + "_fwd")(*inputs, **options, high_precision_level=level)
    gen = torch.Generator().manual_seed(3)
    dy = torch.randn(y.shape, generator=gen).to(cuda_device, dtype)
    grads = getattr(xattn, name + "_bwd")(dy, *inputs, y, lse, **options, high_precision_level=level)[:3]
    refs = [t.detach().double().cpu().requires_grad_() for t in inputs]
    inc, _ = O.allowed_masks(17, 33, 1, operation, 16)
    expected = O.attention_from_mask(*refs, inc, dims[0] ** -0.5)
    want = torch.autograd.grad(expected, refs, dy.double().cpu())
    for g_, w_ in zip(grads, want):
        assert g_.dtype == dtype and torch.isfinite(g_).all()
        assert (g_.double().cpu() - w_).norm() <= 0.015 * w_.norm() + 1e-6


def test_plan_orders_key_tiles_longest_first(cuda_device):
    """The last section of the mask plan lists the key tiles of all batch rows by the number of query
    tiles that see them, most first (the dK / dV kernel starts its CTAs in that order)."""
    from xattn_b200 import _native
    dev = cuda_device
    B, L = 3, 1000
    gen = torch.Generator().manual_seed(3)
    ids = torch.zeros(B, L, dtype=torch.int64)
    for b in range(B):
        pos, seg = 0, 0
        while pos < L:
            n = int(torch.randint(50, 400, (1,), generator=gen))
            ids[b, pos:pos + n] = seg
            pos += n
            seg += 1
    ids = ids.to(dev)
    plan = _native.build_plan(B, L, L, dev, q_segment_idx=ids, k_segment_idx=ids).cpu()
    n_tiles = (L + 127) // 128
    r4 = (B * L + 3) // 4 * 4
    off_kt = 2 * r4 + 4 * B * n_tiles
    off_ko = off_kt + (2 * B * n_tiles + 3) // 4 * 4
    k_tiles = plan[off_kt:off_kt + 2 * B * n_tiles].view(B * n_tiles, 2)
    order = plan[off_ko:off_ko + B * n_tiles]
    assert sorted(order.tolist()) == list(range(B * n_tiles))
    work = (k_tiles[:, 1] - k_tiles[:, 0]).clamp_min(0)[order.long()]
    assert bool((work[1:] <= work[:-1]).all())
    assert int(work[0]) > int(work[-1])


def test_training_step_runs_as_a_cuda_graph(cuda_device):
    """Forward + backward with segment ids captured in a CUDA graph and replayed on new inputs."""
    B, L, Hq, Hkv, D = 2, 640, 8, 2, 128
    gen = torch.Generator().manual_seed(3)
    mk = lambda *s: torch.randn(s, generator=gen).to(device=cuda_device, dtype=torch.bfloat16)
    q, k, v, dy = mk(B, L, Hq, D), mk(B, L, Hkv, D), mk(B, L, Hkv, D), mk(B, L, Hq, D)
    ids = (torch.arange(L, device=cuda_device) // 250).expand(B, -1).contiguous()

    def step():
        y, lse = xattn.causal_flash_attn_fwd(q, k, v, segment_idx=ids)
        return (y, *xattn.causal_flash_attn_bwd(dy, q, k, v, y, lse, segment_idx=ids)[:3])

    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream(cuda_device).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    for t in (q, k, v, dy):
        t.copy_(mk(*t.shape))
    graph.replay()
    eager = step()
    for a, b in zip(outs, eager):
        assert torch.equal(a, b)
    xattn.check_status()


@pytest.mark.parametrize("operation", ("causal_flash_attn", "flash_swa", "flash_sca"))
def test_level1_autograd_equals_standalone_backward(operation, cuda_device):
    """The autograd path reuses the level-1 forward's statistics, the standalone backward recomputes them:
    both give the same bits."""
    B, L, Hq, Hkv, D = 2, 389, 4, 2, 64
    gen = torch.Generator().manual_seed(9)
    mk = lambda *s: torch.randn(s, generator=gen).to(device=cuda_device, dtype=torch.bfloat16)
    q, k, v, dy = mk(B, L, Hq, D), mk(B, L, Hkv, D), mk(B, L, Hkv, D), mk(B, L, Hq, D)
    ids = (torch.arange(L, device=cuda_device) // 150).expand(B, -1).contiguous()
    extra = {"causal_flash_attn": {}, "flash_swa": {"window_size": 100}, "flash_sca": {"chunk_size": 64}}[operation]
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    y = getattr(xattn, operation)(*leaves, **extra, segment_idx=ids, high_precision_level=1)
    grads = torch.autograd.grad(y, leaves, dy)
    y2, lse = getattr(xattn, operation + "_fwd")(q, k, v, **extra, segment_idx=ids, high_precision_level=1)
    assert torch.equal(y, y2)
    alone = getattr(xattn, operation + "_bwd")(dy, q, k, v, y2, lse, **extra, segment_idx=ids, high_precision_level=1)
    for a, b in zip(grads, alone[:3]):
        assert torch.equal(a, b)
    # the standalone backward does not trust what it is given: level-0 statistics give the same result
    y0, lse0 = getattr(xattn, operation + "_fwd")(q, k, v, **extra, segment_idx=ids, high_precision_level=0)
    other = getattr(xattn, operation + "_bwd")(dy, q, k, v, y0, lse0, **extra, segment_idx=ids, high_precision_level=1)
    for a, b in zip(grads, other[:3]):
        assert torch.equal(a, b)


def test_partial_output_merge_kernel(cuda_device):
    """The ring's merge of normalised partial outputs by their lse (one kernel, in place) against the same
    formula in torch, including rows one side or neither side has a key for, and a row offset."""
    from xattn_b200 import _native, parallel as P
    gen = torch.Generator().manual_seed(3)
    B, L, H, V, start = 2, 300, 4, 96, 116
    mk = lambda *s: torch.randn(s, generator=gen).to(cuda_device)
    y0, l0 = mk(B, L, H, V), mk(B, H, L) * 3
    y1, l1 = mk(B, L - start, H, V), mk(B, H, L - start) * 3
    l0[:, :, 5] = float("-inf"); y0[:, 5] = 0            # no key so far
    l1[:, :, 7] = float("-inf"); y1[:, 7] = 0            # no key in this block
    l0[:, :, start + 9] = float("-inf"); y0[:, start + 9] = 0
    l1[:, :, 9] = float("-inf"); y1[:, 9] = 0            # neither
    want_y, want_l = y0.clone(), l0.clone()
    my, ml = P._merge((want_y[:, start:], want_l[:, :, start:]), y1, l1)
    want_y[:, start:], want_l[:, :, start:] = my, ml
    got_y, got_l = y0.clone(), l0.clone()
    _native.merge_partial_outputs(got_y, got_l, y1, l1, start)
    torch.testing.assert_close(got_y, want_y, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(got_l, want_l, atol=1e-6, rtol=1e-6)
    assert torch.equal(got_y[:, :start], y0[:, :start])
    assert torch.isinf(got_l[:, :, start + 9]).all() and torch.count_nonzero(got_y[:, start + 9]) == 0


@pytest.mark.parametrize("level", (0, 1))
def test_backward_in_phases_gives_the_same_bits(level, cuda_device):
    """dK / dV first and dQ in a second call (the order sequence sharding uses to send the halo's gradients
    while the dQ kernel runs) against the one-call backward."""
    from xattn_b200 import _lib, _native
    gen = torch.Generator().manual_seed(17)
    B, Lq, Lk, H, Hkv, D = 2, 300, 428, 4, 2, 128
    mk = lambda *s: torch.randn(s, generator=gen).to(cuda_device, torch.bfloat16)
    q, k, v, dy = mk(B, Lq, H, D), mk(B, Lk, Hkv, D), mk(B, Lk, Hkv, D), mk(B, Lq, H, D)
    plan = _native.build_plan(B, Lq, Lk, cuda_device, visibility="window", span=77)
    out = _native.attention_fwd(q, k, v, plan, D ** -0.5, high_precision=bool(level), return_anchor=bool(level))
    y, lse = out[0], out[1]
    anchor = out[2] if level else None
    whole = _native.BackwardCall(dy, q, k, v, y, lse, plan, D ** -0.5, anchor=anchor).run()
    split = _native.BackwardCall(dy, q, k, v, y, lse, plan, D ** -0.5, anchor=anchor)
    split.dq.fill_(float("nan"))
    split.run(_lib.BWD_PHASE_PRE | _lib.BWD_PHASE_DKV)
    torch.cuda.synchronize()
    assert torch.equal(split.dk, whole.dk) and torch.equal(split.dv, whole.dv)
    assert torch.isnan(split.dq).all()                  # not touched yet
    split.run(_lib.BWD_PHASE_DQ)
    assert torch.equal(split.dq, whole.dq)
    xattn.check_status()
