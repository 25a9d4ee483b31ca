"""The mask-plan cache (the reference's inference BOS forward-plan cache,
csrc/flash_sca/sliding_chunk_attention.cc:113-518): repeated masks reuse their plan, changed masks do not."""
import pytest
import torch

import xattn_b200 as xattn
from xattn_b200.ops import _core

pytestmark = pytest.mark.gpu


def _inputs(dev, B=2, L=700, H=4, Hkv=1, D=64):
    gen = torch.Generator().manual_seed(5)
    mk = lambda *s: torch.randn(s, generator=gen).to(dev, torch.float16)
    return mk(B, L, H, D), mk(B, L, Hkv, D), mk(B, L, Hkv, D)


def test_repeated_bos_mask_reuses_ids_and_plan(cuda_device):
    q, k, v = _inputs(cuda_device)
    bos = torch.zeros(2, 700, dtype=torch.bool, device=cuda_device)
    bos[:, ::190] = True
    xattn.clear_plan_cache()
    with torch.no_grad():
        y0, lse0 = xattn.flash_sca_fwd(q, k, v, 128, bos_mask=bos)
        h0, m0 = _core.plan_cache_stats()
        y1, lse1 = xattn.flash_sca_fwd(q, k, v, 128, bos_mask=bos)
        h1, m1 = _core.plan_cache_stats()
    assert (h1 - h0, m1 - m0) == (2, 0)            # the ids of the mask and the plan built from them
    assert torch.equal(y0, y1) and torch.equal(lse0, lse1)
    # a write into the mask is seen (version counter): new ids, new plan, different result
    bos[:, 95] = True
    with torch.no_grad():
        y2, _ = xattn.flash_sca_fwd(q, k, v, 128, bos_mask=bos)
    h2, m2 = _core.plan_cache_stats()
    assert m2 - m1 == 2
    assert not torch.equal(y1, y2)
    # the uncached result of the same call
    xattn.clear_plan_cache()
    with torch.no_grad():
        y3, _ = xattn.flash_sca_fwd(q, k, v, 128, bos_mask=bos)
    assert torch.equal(y2, y3)
    xattn.check_status()


def test_plans_are_shared_in_training_too(cuda_device):
    q, k, v = _inputs(cuda_device)
    xattn.clear_plan_cache()
    h0, m0 = _core.plan_cache_stats()
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    xattn.flash_swa(*leaves, 100)
    y = xattn.flash_swa(*leaves, 100)
    h1, m1 = _core.plan_cache_stats()
    assert (h1 - h0, m1 - m0) == (1, 1)
    ids = (torch.arange(700, device=cuda_device) // 300).expand(2, -1).contiguous()
    xattn.flash_swa(*leaves, 100, segment_idx=ids)
    y_ids = xattn.flash_swa(*leaves, 100, segment_idx=ids)
    h2, m2 = _core.plan_cache_stats()
    assert (h2 - h1, m2 - m1) == (1, 1)
    ids[:, 350:] += 1                               # a write bumps the version: the old plan is not reused
    y_new = xattn.flash_swa(*leaves, 100, segment_idx=ids)
    assert _core.plan_cache_stats() == (h2, m2 + 1)
    assert not torch.equal(y_ids, y_new) and not torch.equal(y, y_ids)
    # the backward uses the plan its forward saved, whatever the cache holds by then
    xattn.clear_plan_cache()
    grads = torch.autograd.grad(y_new, leaves, torch.ones_like(y_new))
    assert all(torch.isfinite(g).all() for g in grads)
    xattn.check_status()


def test_cache_can_be_switched_off(cuda_device, monkeypatch):
    q, k, v = _inputs(cuda_device)
    monkeypatch.setenv("XATTN_B200_PLAN_CACHE", "0")
    before = _core.plan_cache_stats()
    with torch.no_grad():
        xattn.causal_flash_attn_fwd(q, k, v)
        xattn.causal_flash_attn_fwd(q, k, v)
    assert _core.plan_cache_stats() == before
