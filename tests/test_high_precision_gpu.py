"""Known-answer tests of high_precision_level=1, following the reference's own
(tests/test_high_precision.py:278-310 tiny probability x huge dP, :313-350 constant keys inside segments,
:352-368 rows anchored on one sink key stay bitwise repeatable, :204 long deterministic segments), plus
direct checks of the anchor keys the high-precision forward hands to the backward."""
import math

import pytest
import torch

import xattn_b200 as xattn
from oracle import attention_oracle as O
from tests.test_attention_gpu import assert_grads, assert_output
from xattn_b200 import _native
from xattn_b200.ops import _core

pytestmark = pytest.mark.gpu

OPS = {"full": "causal_flash_attn", "window": "flash_swa", "chunk": "flash_sca"}


@pytest.mark.parametrize("deterministic", (False, True))
@pytest.mark.parametrize("operation", ("full", "chunk"))
def test_tiny_probability_large_value(deterministic, operation, cuda_device):
    """A tiny P times a huge dP is representable and must not vanish early: key 0 holds nearly all of the
    probability of every row that sees it (its logit is 100 above the others), V is ~1e35, so the other
    keys' dS = P dP is ~1e-8 and dQ is the exact negative of their sum.  Bound: 1 % of the gradient's
    norm, the reference's own (tests/test_high_precision.py:309)."""
    torch.manual_seed(31415)
    n, d = 257, 64
    dev = cuda_device
    q = torch.zeros(1, n, 2, d, device=dev, dtype=torch.bfloat16)
    k = torch.zeros(1, n, 1, d, device=dev, dtype=torch.bfloat16)
    q[..., 0] = 1
    k[:, 0, :, 0] = 100 * d ** .5
    v = (torch.randn_like(k, dtype=torch.float32) * 1e35).to(k.dtype)
    g = torch.randn_like(q)
    Q, K, V, G = [t.double().transpose(1, 2) for t in (q, k, v, g)]
    K, V = K.repeat_interleave(2, 1), V.repeat_interleave(2, 1)
    i = torch.arange(n, device=dev)
    mask = i[None, :] <= i[:, None]
    if operation == "chunk":
        mask &= i[None, :] >= ((i[:, None] // 128 - 1) * 128).clamp_min(0)
    p = (Q @ K.transpose(-1, -2) * d ** -.5).masked_fill(~mask, -torch.inf).softmax(-1)
    dp = G @ V.transpose(-1, -2)
    centered = dp - dp.gather(-1, p.argmax(-1, keepdim=True))
    ds = p * (centered - (p * centered).sum(-1, keepdim=True))
    refs = ((ds @ K * d ** -.5).transpose(1, 2),
            (ds.transpose(-1, -2) @ Q * d ** -.5).sum(1, keepdim=True).transpose(1, 2),
            (p.transpose(-1, -2) @ G).sum(1, keepdim=True).transpose(1, 2))
    inputs = [t.requires_grad_() for t in (q, k, v)]
    options = dict(chunk_size=128) if operation == "chunk" else {}
    y = getattr(xattn, OPS[operation])(*inputs, **options, backend="sm90", deterministic=deterministic,
                                       high_precision_level=1)
    grads = torch.autograd.grad(y, inputs, g)
    xattn.check_status()
    for name, actual, ref in zip(("dq", "dk", "dv"), grads, refs):
        assert actual.dtype == torch.bfloat16 and torch.isfinite(actual).all(), name
        assert ref.norm() > 0
        assert (actual.double() - ref).norm() <= .01 * ref.norm(), name
    again = torch.autograd.grad(getattr(xattn, OPS[operation])(
        *inputs, **options, backend="sm90", deterministic=deterministic, high_precision_level=1), inputs, g)
    for a, b in zip(grads, again):
        assert torch.equal(a, b)


@pytest.mark.parametrize("operation,reset", (("full", False), ("window", False), ("chunk", False), ("chunk", True)))
def test_segment_constant_keys(operation, reset, cuda_device):
    """Every query's visible keys are one repeated vector (ones in the first segment, zeros in the others),
    so dQ is exactly zero however large dO V^T is (tests/test_high_precision.py:313-350)."""
    torch.manual_seed(927)
    n, d = 257, 64
    dev = cuda_device
    q = torch.ones(1, n, 2, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.zeros(1, n, 1, d, device=dev, dtype=q.dtype)
    k[:, :128] = 1
    v = (torch.randn_like(k, dtype=torch.float32) * 1e30).to(q.dtype)
    g = torch.randn_like(q)
    ids = (torch.arange(n, device=dev) // 128)[None]
    options = {"window": dict(window_size=64),
               "chunk": dict(chunk_size=64, reset_chunk_pos_per_seq=reset)}.get(operation, {})
    y = getattr(xattn, OPS[operation])(q, k, v, **options, segment_idx=ids, backend="sm90", high_precision_level=1)
    dq, = torch.autograd.grad(y, q, g)
    xattn.check_status()
    assert torch.count_nonzero(dq) == 0


def _llm_like_inputs(dtype, device, n=700, d=64, heads=4):
    """A shared query direction and a sink key at position 0: thousands of rows anchored on one key."""
    gen = torch.Generator(device="cpu").manual_seed(7)
    u = torch.nn.functional.normalize(torch.randn(d, generator=gen), dim=-1)
    amp = math.sqrt(15.0 * math.sqrt(d))
    q = torch.nn.functional.normalize(torch.randn(1, n, heads, d, generator=gen) / math.sqrt(d) + 0.5 * u, dim=-1) * amp
    k = torch.nn.functional.normalize(torch.randn(1, n, 1, d, generator=gen), dim=-1) * amp
    k[:, 0] = u * amp
    v = torch.nn.functional.silu(torch.randn(1, n, 1, d, generator=gen)) + 0.1
    return [t.to(device=device, dtype=dtype).requires_grad_() for t in (q, k, v)]


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16), ids=("bf16", "fp16"))
def test_sink_anchor_rows(dtype, cuda_device):
    """Hundreds of rows anchored on key 0 (tests/test_high_precision.py:352-368): gradients stay bitwise
    repeatable, deterministic or not, and match the FP64 oracle to 2e-3 (FP16) / 5e-3 (BF16, whose final
    rounding alone is 2e-3 per element) of each gradient's norm; 2e-3 is the bound the reference puts
    between its ordered and unordered reductions.  The sink key's dK sums thousands of rounded terms,
    which an element-wise tolerance does not allow for."""
    inputs = _llm_like_inputs(dtype, cuda_device)
    n = inputs[0].shape[1]
    dy = (torch.randn(1, n, 4, 64, generator=torch.Generator().manual_seed(8)) / n ** 0.5).to(cuda_device, dtype)
    results = []
    for deterministic in (True, True, False):
        out = xattn.causal_flash_attn(*inputs, deterministic=deterministic, high_precision_level=1)
        results.append(torch.autograd.grad(out, inputs, dy))
    xattn.check_status()
    for other in results[1:]:
        for a, b in zip(results[0], other):
            assert torch.equal(a, b)
    # most rows really are anchored on the sink
    _, _, anchor = _native.attention_fwd(*[t.detach() for t in inputs],
                                         _core.make_plan(inputs[0], n, _core.Support("full"), None, None),
                                         64 ** -0.5, high_precision=True, return_anchor=True)
    assert (anchor == 0).float().mean() > 0.5
    refs = [t.detach().double().cpu().requires_grad_() for t in inputs]
    inc, _ = O.allowed_masks(n, n, 1, "full", None)
    yr = O.attention_from_mask(*refs, inc, 64 ** -0.5)
    gr = torch.autograd.grad(yr, refs, dy.double().cpu())
    for got, ref in zip(results[0], gr):
        assert torch.isfinite(got).all()
        assert (got.double().cpu() - ref).norm() <= (2e-3 if dtype == torch.float16 else 5e-3) * ref.norm()


def test_deterministic_long_segments(cuda_device):
    """More key tiles than resident CTAs, level 1, segments of 2048 (tests/test_high_precision.py:204):
    parity on sampled rows against the FP64 oracle and bitwise repeatability."""
    B, L, H, Hkv, D = 4, 4096, 4, 4, 64
    gen = torch.Generator().manual_seed(204)
    mk = lambda *s: torch.randn(s, generator=gen).to(device=cuda_device, dtype=torch.bfloat16)
    q, k, v = mk(B, L, H, D), mk(B, L, Hkv, D), mk(B, L, Hkv, D)
    q, k = [torch.nn.functional.normalize(t.float(), dim=-1).to(torch.bfloat16) for t in (q, k)]
    ids = (torch.arange(L, device=cuda_device) // 2048).expand(B, -1).contiguous()
    rows = torch.tensor([0, 1, 127, 128, 2047, 2048, 3000, 4095])
    dy = torch.zeros(B, L, H, D, device=cuda_device, dtype=torch.bfloat16)
    dy[:, rows] = mk(B, len(rows), H, D) / 8
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    y = xattn.causal_flash_attn(*leaves, segment_idx=ids, deterministic=True, high_precision_level=1)
    grads = torch.autograd.grad(y, leaves, dy)
    y2 = xattn.causal_flash_attn(*leaves, segment_idx=ids, deterministic=True, high_precision_level=1)
    for a, b in zip(grads, torch.autograd.grad(y2, leaves, dy)):
        assert torch.equal(a, b)
    xattn.check_status()
    # oracle on the sampled rows only: queries = those rows, keys = everything
    qs = q[:, rows].double().cpu().requires_grad_()
    kr, vr = [t.double().cpu().requires_grad_() for t in (k, v)]
    pos = rows[None, :, None]
    kpos = torch.arange(L)[None, None, :]
    inc = ((kpos <= pos) & (ids.cpu()[:, rows][:, :, None] == ids.cpu()[:, None, :]))
    yr = O.attention_from_mask(qs, kr, vr, inc, D ** -0.5)
    gq, gk, gv = torch.autograd.grad(yr, (qs, kr, vr), dy[:, rows].double().cpu())
    assert_output(y[:, rows].detach(), yr.detach(), torch.bfloat16)
    assert_grads([grads[0][:, rows], grads[1], grads[2]], [gq, gk, gv], torch.bfloat16)


def test_forward_anchor_is_first_argmax(cuda_device):
    """The anchor the high-precision forward returns is the first visible key with the row's largest logit,
    -1 for a row without keys."""
    B, Lq, Lk, H, Hkv, D = 2, 300, 421, 4, 2, 64
    gen = torch.Generator().manual_seed(3)
    mk = lambda *s: torch.randn(s, generator=gen).to(device=cuda_device, dtype=torch.bfloat16)
    q, k, v = mk(B, Lq, H, D), mk(B, Lk, Hkv, D), mk(B, Lk, Hkv, D)
    k[:, 50:60] = k[:, 50:51]                       # ties: ten identical keys
    ki = (torch.arange(Lk, device=cuda_device) // 97).expand(B, -1).contiguous()
    qi = ki[:, -Lq:].clone()
    qi[:, :5] = -1                                  # rows without keys
    plan = _core.make_plan(q, Lk, _core.Support("window", 120), qi, ki)
    _, lse, anchor = _native.attention_fwd(q, k, v, plan, D ** -0.5, high_precision=True, return_anchor=True)
    xattn.check_status()
    inc, _ = O.allowed_masks(Lq, Lk, B, "window", 120, qi.cpu(), ki.cpu(), False)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float().cpu(), k.float().cpu().repeat_interleave(H // Hkv, 2))
    s = s.masked_fill(~inc[:, None], -torch.inf)
    expect = s.argmax(-1).to(torch.int32)
    expect[~inc.any(-1)[:, None].expand_as(expect)] = -1
    got = anchor.cpu()
    # FP32 accumulation order differs between the tensor core and the CPU: accept any key whose logit equals
    # the row maximum to within rounding, and demand the first of exactly equal keys on the tie block
    picked = s.gather(-1, got.clamp_min(0).long()[..., None]).squeeze(-1)
    best = s.max(-1).values
    live = expect >= 0
    assert torch.equal(got < 0, ~live)
    assert torch.all((best - picked)[live].abs() <= 1e-3 * best[live].abs().clamp_min(1))
    in_tie = live & (got >= 50) & (got < 60)
    assert torch.all(got[in_tie] == 50)
