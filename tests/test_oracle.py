"""The CPU oracle against golden outputs of the reference's own oracle (tests/golden), and the
interval property the device plan relies on."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from golden_cases import GOLDEN_CASES, golden_inputs  # noqa: E402

from oracle import attention_oracle as O  # noqa: E402
from tests._cases import cases_for, metadata_for  # noqa: E402

GOLDEN = np.load(os.path.join(HERE, "golden", "attention_golden.npz"))


@pytest.mark.parametrize("case", GOLDEN_CASES, ids=lambda c: c["name"])
def test_oracle_matches_reference_golden(case):
    t = golden_inputs(case)
    name = case["name"]
    inc, strict = O.allowed_masks(case["Lq"], case["Lk"], case["B"], case["vis"], case["span"],
                                  t["q_ids"], t["k_ids"], case["reset"])
    shape = (case["B"], case["Lq"], case["Lk"])
    n = int(np.prod(shape))
    for mine, key in ((inc, "inclusive"), (strict, "strict")):
        ref = np.unpackbits(GOLDEN[f"{name}/{key}"])[:n].reshape(shape).astype(bool)
        assert np.array_equal(mine.numpy(), ref), f"{key} mask differs from the reference's"
    q, k, v = (t[x].clone().requires_grad_() for x in ("q", "k", "v"))
    y = O.attention_from_mask(q, k, v, strict if case["strict"] else inc, case["D"] ** -0.5)
    grads = torch.autograd.grad(y, (q, k, v), t["dy"])
    for val, key in zip((y, *grads), ("y", "dq", "dk", "dv")):
        np.testing.assert_allclose(val.detach().numpy(), GOLDEN[f"{name}/{key}"], rtol=1e-12, atol=1e-13)
    if case["softdelta"]:
        q, k, v, g = (t[x].clone().requires_grad_() for x in ("q", "k", "v", "g"))
        dy = t["dy"]
        if case.get("groups"):
            shape = (case["groups"], case["V"] // case["groups"])
            v = t["v"].unflatten(3, shape).clone().requires_grad_()
            dy = dy.unflatten(3, shape)
        ys, _, _ = O.softdelta(q, k, v, g, None, scale=case["D"] ** -0.5, q_segment_idx=t["q_ids"],
                               k_segment_idx=t["k_ids"], visibility=case["vis"], span=case["span"],
                               reset_position_per_segment=case["reset"])
        gs = torch.autograd.grad(ys, (q, k, v, g), dy)
        for val, key in zip((ys, *gs), ("sd_y", "sd_dq", "sd_dk", "sd_dv", "sd_dg")):
            np.testing.assert_allclose(val.detach().numpy(), GOLDEN[f"{name}/{key}"], rtol=1e-12, atol=1e-13)


@pytest.mark.parametrize("operation", ("full", "window", "chunk"))
@pytest.mark.parametrize("strict", (False, True))
def test_visible_keys_form_one_interval(operation, strict):
    """Every case of the parity matrix: a row's visible keys are contiguous (row_intervals asserts it)
    and the interval reproduces the mask."""
    for case in cases_for(operation):
        if case.q_length * (case.k_length + case.previous) > 80000:
            continue
        _, qi, ki = metadata_for(case, torch.device("cpu"))
        total = case.k_length + case.previous
        lo, hi = O.row_intervals(case.q_length, total, case.batch, operation, case.span, qi, ki, case.reset, strict)
        inc, st = O.allowed_masks(case.q_length, total, case.batch, operation, case.span, qi, ki, case.reset)
        mask = st if strict else inc
        idx = torch.arange(total)[None, None, :]
        rebuilt = (idx >= lo[:, :, None]) & (idx < hi[:, :, None])
        assert torch.equal(rebuilt, mask), case.name


def test_empty_rows_read_zero():
    q = torch.randn(1, 3, 2, 8, dtype=torch.float64)
    k = torch.randn(1, 5, 1, 8, dtype=torch.float64)
    v = torch.randn(1, 5, 1, 8, dtype=torch.float64)
    mask = torch.zeros(1, 3, 5, dtype=torch.bool)
    mask[0, 2, :2] = True
    y = O.attention_from_mask(q, k, v, mask, 0.3)
    assert torch.count_nonzero(y[:, :2]) == 0 and torch.isfinite(y).all()
    lse = O.lse_from_mask(q, k, mask, 0.3)
    assert torch.isinf(lse[0, :, :2]).all() and torch.isfinite(lse[0, :, 2]).all()


def test_visible_pair_count_causal():
    lo, hi = O.row_intervals(1024, 1024, 1, "full", None)
    assert O.visible_pairs(lo, hi) == 1024 * 1025 // 2
    lo, hi = O.row_intervals(64, 64, 1, "window", 7)
    assert O.visible_pairs(lo, hi) == sum(min(i, 7) + 1 for i in range(64))
    lo, hi = O.row_intervals(64, 64, 1, "chunk", 8)
    assert O.visible_pairs(lo, hi) == sum(i - max(0, (i // 8 - 1) * 8) + 1 for i in range(64))


def _compiled_reference():
    from oracle import build_ref
    return build_ref.load("_reference"), build_ref.load("reference")


@pytest.mark.parametrize("operation", ("full", "window", "chunk"))
def test_port_matches_compiled_reference(operation):
    """oracle/_ref holds the reference's own oracle compiled from its sources (oracle/build_ref.py): on
    the whole parity matrix the restatement gives the same masks bit for bit and the same reads and
    gradients to FP64 rounding.  Skipped where oracle/_ref has not been built."""
    ref, _ = _compiled_reference()
    if ref is None:
        pytest.skip("oracle/_ref not built (python oracle/build_ref.py <reference root>)")
    from tests._cases import make_inputs
    cpu = torch.device("cpu")
    for case in cases_for(operation):
        total = case.k_length + case.previous
        if case.q_length * total > 80000:
            continue
        _, qi, ki = metadata_for(case, cpu)
        mine = O.allowed_masks(case.q_length, total, case.batch, operation, case.span, qi, ki, case.reset)
        theirs = ref._allowed_masks(case.q_length, total, case.batch, cpu, operation, case.span, qi, ki, case.reset)
        for a, b in zip(mine, theirs):
            assert torch.equal(a, b.expand_as(a)), case.name
        inputs = make_inputs(operation, case, torch.bfloat16, 2, cpu)
        q, k, v = (t.detach().double() for t in inputs[:3])
        if case.previous:
            k = torch.cat((inputs[-2].detach().double(), k), 1)
            v = torch.cat((inputs[-1].detach().double(), v), 1)
        outs = []
        for read in (O.attention_from_mask, ref._attention_from_mask):
            leaves = [t.clone().requires_grad_() for t in (q, k, v)]
            y = read(*leaves, mine[0], case.dim ** -0.5)
            dy = torch.randn(y.shape, generator=torch.Generator().manual_seed(5), dtype=torch.float64)
            outs.append((y.detach(), *torch.autograd.grad(y, leaves, dy)))
        for a, b in zip(*outs):
            torch.testing.assert_close(a, b, rtol=1e-12, atol=1e-13)


def test_softdelta_port_matches_compiled_reference():
    _, ref = _compiled_reference()
    if ref is None:
        pytest.skip("oracle/_ref not built (python oracle/build_ref.py <reference root>)")
    gen = torch.Generator().manual_seed(12)
    B, L, H, Hkv, D, V = 2, 37, 4, 2, 16, 24
    mk = lambda *s: torch.randn(s, generator=gen, dtype=torch.float64)
    q, k, v, g = mk(B, L, H, D), mk(B, L, Hkv, D), mk(B, L, Hkv, V), mk(B, L, H)
    ids = (torch.arange(L) // 11).expand(B, -1).contiguous()
    for vis, span in (("full", None), ("window", 5), ("chunk", 8)):
        kw = dict(scale=0.3, q_segment_idx=ids, k_segment_idx=ids, visibility=vis, span=span)
        mine = O.softdelta(q, k, v, g, None, **kw)[0]
        theirs = ref.softdelta_fp64_oracle(q, k, v, g, None, **kw)
        theirs = theirs[0] if isinstance(theirs, tuple) else theirs
        torch.testing.assert_close(mine, theirs, rtol=1e-12, atol=1e-13)


def test_hand_written_gradients_of_the_bounds_helper():
    """tests/_bounds.py writes the read's gradients out by hand (to get at the magnitudes its tolerances
    scale with): they equal autograd of the oracle, and every magnitude is at least the value."""
    from tests._bounds import read_with_scales
    gen = torch.Generator().manual_seed(21)
    B, R, Lk, H, Hkv, D, V = 2, 7, 33, 4, 2, 16, 24
    mk = lambda *s: torch.randn(s, generator=gen, dtype=torch.float64)
    q, k, v, dy = mk(B, R, H, D), mk(B, Lk, Hkv, D), mk(B, Lk, Hkv, V), mk(B, R, H, V)
    rows = torch.tensor([0, 3, 9, 10, 20, 31, 32])
    ids = (torch.arange(Lk) // 10).expand(B, -1).contiguous()
    mask, _ = O.allowed_masks(Lk, Lk, B, "window", 6, ids, ids, False, rows=rows)
    mask[:, 2] = False                        # a row without keys
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    y = O.attention_from_mask(*leaves, mask, 0.25)
    grads = torch.autograd.grad(y, leaves, dy)
    got = read_with_scales(q, k, v, mask, dy, 0.25)
    for a, b in zip((got.y, got.dq, got.dk, got.dv), (y.detach(), *grads)):
        torch.testing.assert_close(a, b, rtol=1e-12, atol=1e-13)
    for val, mag in ((got.y, got.y_scale), (got.dq, got.dq_scale), (got.dk, got.dk_scale), (got.dv, got.dv_scale)):
        assert torch.all(mag + 1e-15 >= val.abs())
