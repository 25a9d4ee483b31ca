"""Parity at the benchmark configurations themselves: exact shape, dtype, head layout, span and
packing of BASELINE.json configs[1]-[4], levels 0 and 1 where the configuration names both.

The FP64 oracle cannot hold a whole 8192 x 8192 (or 32768 x 32768) score matrix per head, so the method
is the reference's own for long sequences (tests/_numerics.py:293-320): a few sampled query rows per
batch row against ALL keys, with dO nonzero on those rows only.  y and dq are compared on the sampled
rows (dq must be exactly zero elsewhere), dk and dv on the full tensors, element by element with the
reference's ATOL / GRAD_ATOL and RTOL (tests/_reference.py:7-20), RTOL applied to the magnitude an
element's rounding errors scale with (tests/_bounds.py says why N(0,1) inputs need that).
Inputs are seeded synthetic tensors with the configurations' distributions.
"""
import pytest
import torch

import xattn_b200 as xattn
from oracle import attention_oracle as O
from tests._bounds import assert_within, read_with_scales

pytestmark = pytest.mark.gpu


def _draw(gen, std, dtype, device, *shape):
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(device=device, dtype=dtype)


def _segment_ids(gen, batch, length, lo, hi):
    """Segments of length ~U[lo, hi] laid end to end, the last one cut at the sequence end; int64 ids."""
    ids = torch.zeros(batch, length, dtype=torch.int64)
    for b in range(batch):
        pos = seg = 0
        while pos < length:
            n = int(torch.randint(lo, hi + 1, (1,), generator=gen))
            ids[b, pos:pos + n] = seg
            pos += n
            seg += 1
    return ids


def _sample_rows(gen, ids, length, extra=()):
    """Rows at segment starts and ends, tile edges, and a few random ones; the same rows for every batch
    row so that the sampled tensors stay rectangular."""
    rows = {0, 1, 127, 128, 129, length // 2, length - 129, length - 2, length - 1, *extra}
    if ids is not None:
        change = (ids[0, 1:] != ids[0, :-1]).nonzero().flatten() + 1
        for c in change[:3].tolist():
            rows |= {c - 1, c, c + 1}
    rows |= set(torch.randint(0, length, (4,), generator=gen).tolist())
    return torch.tensor(sorted(r for r in rows if 0 <= r < length))


def _mask_for_rows(rows, length, batch, visibility, span, ids, strict=False):
    inc, past = O.allowed_masks(length, length, batch, visibility, span, ids, ids, False, rows=rows)
    return past if strict else inc


def _check_attention(op, kwargs, q, k, v, rows, dy_rows, mask, level):
    """Public op + autograd on the full tensors against the oracle on the sampled rows."""
    dtype, dev = q.dtype, q.device
    L = q.shape[1]
    rd = rows.to(dev)
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    y = op(*leaves, **kwargs, high_precision_level=level)
    dy = torch.zeros_like(y)
    dy[:, rd] = dy_rows
    dq, dk, dv = torch.autograd.grad(y, leaves, dy)
    xattn.check_status()
    ref = read_with_scales(q[:, rd].double().cpu(), k.double().cpu(), v.double().cpu(), mask,
                           dy_rows.double().cpu(), q.shape[-1] ** -0.5)
    rtol = O.RTOL[dtype]
    assert_within(y[:, rd], ref.y, ref.y_scale, O.ATOL[dtype], rtol, "y")
    assert_within(dq[:, rd], ref.dq, ref.dq_scale, O.GRAD_ATOL[dtype], rtol, "dq")
    assert_within(dk, ref.dk, ref.dk_scale, O.GRAD_ATOL[dtype], rtol, "dk")
    assert_within(dv, ref.dv, ref.dv_scale, O.GRAD_ATOL[dtype], rtol, "dv")
    others = torch.ones(L, dtype=torch.bool)
    others[rows] = False
    assert torch.count_nonzero(dq[:, others.to(dev)]) == 0
    # the gradients of a second run are the same bits
    y2 = op(*leaves, **kwargs, high_precision_level=level)
    for a, b in zip((dq, dk, dv), torch.autograd.grad(y2, leaves, dy)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("level", (0, 1))
def test_config1_causal_gqa_packed_segments(level, cuda_device):
    """configs[1]: causal, bf16, GQA 32/8, B=4, S=8192, D=128, segments ~U[512,4096] as int64 ids."""
    gen = torch.Generator().manual_seed(1)
    B, S, Hq, Hkv, D = 4, 8192, 32, 8, 128
    dt, dev = torch.bfloat16, cuda_device
    q, k, v = _draw(gen, 1.0, dt, dev, B, S, Hq, D), _draw(gen, 1.0, dt, dev, B, S, Hkv, D), _draw(gen, 1.0, dt, dev, B, S, Hkv, D)
    ids = _segment_ids(gen, B, S, 512, 4096)
    rows = _sample_rows(gen, ids, S)
    dy_rows = _draw(gen, 1.0, dt, dev, B, len(rows), Hq, D)
    mask = _mask_for_rows(rows, S, B, "full", None, ids)
    _check_attention(xattn.causal_flash_attn, dict(segment_idx=ids.to(dev)), q, k, v, rows, dy_rows, mask, level)


def test_config2_sliding_window_long(cuda_device):
    """configs[2]: sliding window, bf16, B=1, S=32768, GQA 32/8, D=128, window 4096, one segment."""
    gen = torch.Generator().manual_seed(2)
    B, S, Hq, Hkv, D, W = 1, 32768, 32, 8, 128, 4096
    dt, dev = torch.bfloat16, cuda_device
    q, k, v = _draw(gen, 1.0, dt, dev, B, S, Hq, D), _draw(gen, 1.0, dt, dev, B, S, Hkv, D), _draw(gen, 1.0, dt, dev, B, S, Hkv, D)
    rows = _sample_rows(gen, None, S, extra=(W - 1, W, W + 1, 2 * W, S - W))
    dy_rows = _draw(gen, 1.0, dt, dev, B, len(rows), Hq, D)
    mask = _mask_for_rows(rows, S, B, "window", W, None)
    _check_attention(xattn.flash_swa, dict(window_size=W), q, k, v, rows, dy_rows, mask, 0)


@pytest.mark.parametrize("level", (0, 1))
def test_config3_sliding_chunk_fp16_mqa_bos(level, cuda_device):
    """configs[3]: sliding chunk, fp16, MQA 16/1, B=2, S=16384, D=128, chunk 2048, inputs N(0, 0.5^2),
    BOS-mask packing with a BOS every ~U[1024,8192] tokens."""
    gen = torch.Generator().manual_seed(3)
    B, S, Hq, Hkv, D, C = 2, 16384, 16, 1, 128, 2048
    dt, dev = torch.float16, cuda_device
    q, k, v = _draw(gen, 0.5, dt, dev, B, S, Hq, D), _draw(gen, 0.5, dt, dev, B, S, Hkv, D), _draw(gen, 0.5, dt, dev, B, S, Hkv, D)
    ids = _segment_ids(gen, B, S, 1024, 8192)
    bos = torch.ones(B, S, dtype=torch.bool)
    bos[:, 1:] = ids[:, 1:] != ids[:, :-1]
    rows = _sample_rows(gen, ids, S, extra=(C - 1, C, 2 * C - 1, 2 * C, 2 * C + 1))
    dy_rows = _draw(gen, 0.5, dt, dev, B, len(rows), Hq, D)
    mask = _mask_for_rows(rows, S, B, "chunk", C, ids)
    _check_attention(xattn.flash_sca, dict(chunk_size=C, bos_mask=bos.to(dev)), q, k, v, rows, dy_rows, mask, level)


@pytest.mark.parametrize("level", (0, 1))
@pytest.mark.parametrize("window", (None, 2048), ids=("causal", "window2048"))
def test_config4_softdelta(window, level, cuda_device):
    """configs[4]: SoftDelta and sliding-window SoftDelta, bf16, B=2, S=8192, MHA 16/16, D=128,
    window 2048 for the windowed form, gate logits ~U(0,1), aligned keys as the second reader."""
    gen = torch.Generator().manual_seed(4)
    B, S, H, D = 2, 8192, 16, 128
    dt, dev = torch.bfloat16, cuda_device
    q, k, v = _draw(gen, 1.0, dt, dev, B, S, H, D), _draw(gen, 1.0, dt, dev, B, S, H, D), _draw(gen, 1.0, dt, dev, B, S, H, D)
    g = torch.rand(B, S, H, generator=gen).to(dev, dt)
    extra = () if window is None else (window - 1, window, window + 1)
    rows = _sample_rows(gen, None, S, extra=extra)
    rd = rows.to(dev)
    dy_rows = _draw(gen, 1.0, dt, dev, B, len(rows), H, D)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g)]
    if window is None:
        y = xattn.softdelta_attention(q=leaves[0], k=leaves[1], k_read=None, v=leaves[2], g=leaves[3],
                                      high_precision_level=level)
    else:
        y = xattn.sliding_window_softdelta_attention(q=leaves[0], k=leaves[1], k_read=None, v=leaves[2], g=leaves[3],
                                                     window_size=window, high_precision_level=level)
    dy = torch.zeros_like(y)
    dy[:, rd] = dy_rows
    dq, dk, dv, dg = torch.autograd.grad(y, leaves, dy)
    xattn.check_status()
    # oracle on the sampled rows: y = read(q) - sigmoid(g) * read(aligned key, strict past)
    vis = "full" if window is None else "window"
    inc, strict = O.allowed_masks(S, S, B, vis, window, None, None, False, rows=rows)
    k64, v64 = k.double().cpu(), v.double().cpu()
    gate = torch.sigmoid(g[:, rd].double().cpu())[..., None]
    dyr = dy_rows.double().cpu()
    scale = D ** -0.5
    read = read_with_scales(q[:, rd].double().cpu(), k64, v64, inc, dyr, scale)
    neg = read_with_scales(k64[:, rows], k64, v64, strict, -gate * dyr, scale)      # Hq == Hkv here
    rtol = O.RTOL[dt]
    assert_within(y[:, rd], read.y - gate * neg.y, read.y_scale + gate * neg.y_scale, O.ATOL[dt], rtol, "y")
    assert_within(dq[:, rd], read.dq, read.dq_scale, O.GRAD_ATOL[dt], rtol, "dq")
    # the aligned keys are the second reader's queries: their gradient lands on the sampled rows of dk
    ek, ek_scale = read.dk + neg.dk, read.dk_scale + neg.dk_scale
    ek[:, rows] += neg.dq
    ek_scale[:, rows] += neg.dq_scale
    assert_within(dk, ek, ek_scale, O.GRAD_ATOL[dt], rtol, "dk")
    assert_within(dv, read.dv + neg.dv, read.dv_scale + neg.dv_scale, O.GRAD_ATOL[dt], rtol, "dv")
    # dg = -sigmoid'(g) <dy, neg_read>
    dgate = gate * (1 - gate)
    eg = -(dgate * dyr * neg.y).sum(-1)
    eg_scale = (dgate * dyr.abs() * neg.y_scale).sum(-1)
    assert_within(dg[:, rd], eg, eg_scale, O.GRAD_ATOL[dt], rtol, "dg")
