"""Decode shapes (a few query rows against many keys) on the split forward: the query heads of a KV
group share one tile and the keys are divided among CTAs.  Checked against the CPU oracle through
the public ops (same case runner as the other parity tests, so gradients of the short right-aligned
Q are covered too), against the general kernel for every split count, and on the known answers the
reference pins for level 1 (one visible key returns V bit for bit, tests/test_high_precision.py:89-139)."""
import pytest
import torch

import xattn_b200 as xattn
from xattn_b200 import _lib, _native
from oracle import attention_oracle as O
from tests._cases import Case
from tests.test_attention_gpu import OPS, check_case

pytestmark = pytest.mark.gpu

DECODE_CASES = (
    Case("decode-long", 1, 1000, 64, 64, batch=2),
    Case("decode-dims", 1, 2049, 40, 56, batch=1),
    Case("decode-wide", 1, 777, 256, 160, batch=1),
    Case("speculative", 8, 1536, 128, 128, batch=2),
    Case("speculative-segment", 16, 900, 96, 128, metadata="independent", batch=2),
    Case("speculative-bos", 5, 640, 64, 192, metadata="bos", batch=1),
    Case("decode-empty-rows", 4, 600, 64, 64, metadata="unmatched"),
    Case("decode-head-view", 2, 515, layout="head_slice"),
    Case("decode-strided", 3, 515, layout="last_stride"),
)


def test_library_suggests_splits_for_decode_shapes():
    lib = _lib.load()
    suggest = lib.xattn_b200_fwd_split_suggest
    assert suggest(1, 1, 32768, 32, 8, 148) == 18          # 148 SMs / 8 (batch, KV head) pairs
    assert suggest(64, 1, 32768, 32, 8, 148) == 1          # enough pairs: only the heads are shared
    assert suggest(64, 1, 32768, 8, 8, 148) == 0           # nothing to share, nothing to divide
    assert suggest(1, 1, 1024, 32, 8, 148) == 4            # at least two key tiles per CTA
    assert suggest(1, 1, 300, 32, 8, 148) == 0             # short keys: the general kernel
    assert suggest(1, 33, 32768, 32, 8, 148) == 0          # 33 rows x 4 heads do not fit one tile
    assert suggest(1, 1, 32768, 24, 8, 148) == 0           # group of 3: not a power of two
    assert lib.xattn_b200_fwd_split_workspace_bytes(2, 3, 32, 128, 5) == 5 * 2 * 3 * 32 * 129 * 4


@pytest.mark.parametrize("case", DECODE_CASES, ids=lambda c: c.name)
@pytest.mark.parametrize("operation", OPS)
@pytest.mark.parametrize("kv_heads", (1, 2, 4), ids=("mqa", "gqa", "mha"))
def test_decode_case_matches_oracle(operation, case, kv_heads, cuda_device):
    lib = _lib.load()
    assert lib.xattn_b200_fwd_split_suggest(case.batch, case.q_length, case.k_length, 4, kv_heads, 148) > 0 or kv_heads == 4
    for dtype, level in ((torch.bfloat16, 0), (torch.float16, 0), (torch.bfloat16, 1)):
        check_case(operation, case, dtype, kv_heads, level, cuda_device)


def _decode_inputs(B, Lq, Lk, Hq, Hkv, D, V, dtype, device, seed=5):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, Lq, Hq, D, generator=gen).to(device=device, dtype=dtype)
    k = torch.randn(B, Lk, Hkv, D, generator=gen).to(device=device, dtype=dtype)
    v = torch.randn(B, Lk, Hkv, V, generator=gen).to(device=device, dtype=dtype)
    return q, k, v


@pytest.mark.parametrize("B,Lq,Lk,Hq,Hkv,D,V", (
    (1, 1, 8192, 32, 8, 128, 128),
    (3, 1, 4100, 16, 1, 128, 128),      # MQA: 16 heads in one tile
    (2, 4, 3000, 32, 1, 64, 64),        # 4 rows x 32 heads fill the tile
    (2, 2, 1111, 8, 8, 256, 256),       # MHA: only the keys are divided
    (1, 128, 2048, 4, 4, 128, 96),
))
@pytest.mark.parametrize("visibility,span", (("full", None), ("window", 700), ("chunk", 512)))
def test_every_split_count_agrees_with_the_general_kernel(B, Lq, Lk, Hq, Hkv, D, V, visibility, span, cuda_device):
    dtype = torch.bfloat16
    q, k, v = _decode_inputs(B, Lq, Lk, Hq, Hkv, D, V, dtype, cuda_device)
    plan = _native.build_plan(B, Lq, Lk, cuda_device, visibility=visibility, span=span)
    scale = D ** -0.5
    for level in (False, True):
        y0, lse0 = _native.attention_fwd(q, k, v, plan, scale, high_precision=level, splits=0)
        inc, _ = O.allowed_masks(Lq, Lk, B, visibility, span)
        ref = O.attention_from_mask(q.double().cpu(), k.double().cpu(), v.double().cpu(), inc, scale)
        torch.testing.assert_close(y0.cpu(), ref.to(dtype), atol=O.ATOL[dtype], rtol=O.RTOL[dtype])
        for splits in (1, 2, 3, 7, 16, 64):
            state = torch.empty(B, Lq, Hq, V, dtype=torch.float32, device=cuda_device)
            y, lse = _native.attention_fwd(q, k, v, plan, scale, high_precision=level, splits=splits, output_state=state)
            torch.testing.assert_close(y.cpu(), ref.to(dtype), atol=O.ATOL[dtype], rtol=O.RTOL[dtype])
            torch.testing.assert_close(lse, lse0, atol=2e-5, rtol=1e-5)
            torch.testing.assert_close(y.float(), y0.float(), atol=1e-2, rtol=1e-2)
            assert torch.equal(state.to(dtype), y)
            y_again, lse_again = _native.attention_fwd(q, k, v, plan, scale, high_precision=level, splits=splits)
            assert torch.equal(y, y_again) and torch.equal(lse, lse_again), "bitwise repeatable"
    _native.check_status()


def test_single_visible_key_returns_value_exactly(cuda_device):
    """Level 1, window 0: every row sees exactly its own key, whichever split holds it."""
    B, Lq, Lk, Hq, Hkv, D = 2, 3, 2000, 8, 2, 128
    q, k, v = _decode_inputs(B, Lq, Lk, Hq, Hkv, D, D, torch.bfloat16, cuda_device)
    y = xattn.flash_swa(q, k, v, window_size=0, high_precision_level=1)
    own = v[:, Lk - Lq:].repeat_interleave(Hq // Hkv, dim=2)
    assert torch.equal(y, own)
    y, lse = xattn.flash_swa_fwd(q, k, v, window_size=0, high_precision_level=1)
    assert torch.equal(y, own)
    s = (q.float() * k[:, Lk - Lq:].repeat_interleave(Hq // Hkv, dim=2).float()).sum(-1) * D ** -0.5
    torch.testing.assert_close(lse, s.transpose(1, 2), atol=1e-4, rtol=1e-5)


def test_rows_without_keys_and_segments(cuda_device):
    """Key segment ids that no query carries: y = 0, lse = -inf from every split."""
    B, Lq, Lk, Hq, Hkv, D = 1, 2, 1500, 8, 2, 64
    q, k, v = _decode_inputs(B, Lq, Lk, Hq, Hkv, D, D, torch.float16, cuda_device)
    q_ids = torch.full((B, Lq), 7, dtype=torch.int64, device=cuda_device)
    k_ids = torch.zeros((B, Lk), dtype=torch.int64, device=cuda_device)
    y, lse = xattn.causal_flash_attn_fwd(q, k, v, q_segment_idx=q_ids, k_segment_idx=k_ids)
    assert torch.count_nonzero(y) == 0 and torch.isinf(lse).all() and (lse < 0).all()
    # the last 300 keys belong to the queries' segment: only they count
    k_ids[:, -300:] = 7
    y, lse = xattn.causal_flash_attn_fwd(q, k, v, q_segment_idx=q_ids, k_segment_idx=k_ids)
    y_ref, lse_ref = xattn.causal_flash_attn_fwd(q, k[:, -300:], v[:, -300:])
    torch.testing.assert_close(y.float(), y_ref.float(), atol=2e-3, rtol=1e-2)
    torch.testing.assert_close(lse, lse_ref, atol=1e-4, rtol=1e-5)


def test_split_entry_rejects_bad_arguments(cuda_device):
    q, k, v = _decode_inputs(1, 64, 1024, 8, 2, 64, 64, torch.bfloat16, cuda_device)
    plan = _native.build_plan(1, 64, 1024, cuda_device)
    with pytest.raises(RuntimeError, match="q_len"):
        _native.attention_fwd(q, k, v, plan, 0.125, splits=2)     # 64 rows x 4 heads > 128
    q = q[:, :2]
    plan = _native.build_plan(1, 2, 1024, cuda_device)
    with pytest.raises(RuntimeError, match="splits"):
        _native.attention_fwd(q, k, v, plan, 0.125, splits=1000)


@pytest.mark.parametrize("q_length", (1, 4))
@pytest.mark.parametrize("heads", ((8, 2), (4, 4), (16, 1)), ids=("gqa", "mha", "mqa"))
@pytest.mark.parametrize("variant", ("causal", "window", "chunk"))
@pytest.mark.parametrize("level", (0, 1))
def test_softdelta_decode_shapes(q_length, heads, variant, level, cuda_device):
    """Both reads of SoftDelta (the query read and the strict-past read of k_read) on the split forward."""
    from tests.test_softdelta_gpu import check, make_inputs
    dtype = torch.bfloat16
    t = make_inputs(cuda_device, dtype, 2, 900, heads[0], heads[1], 64, 128, True, q_length=q_length, seed=13)
    if variant == "causal":
        check("softdelta_attention", t, dtype, level)
    elif variant == "window":
        check("sliding_window_softdelta_attention", t, dtype, level, dict(window_size=600),
              dict(visibility="window", span=600))
    else:
        check("sliding_chunk_softdelta_attention", t, dtype, level, dict(chunk_size=512),
              dict(visibility="chunk", span=512))


def test_decode_step_runs_as_a_cuda_graph(cuda_device):
    """Plan, split forward and merge kernel captured once and replayed on new inputs (the launch-bound
    serving loop): the device-status protocol makes no event queries during capture."""
    B, Lk, Hq, Hkv, D = 2, 4096, 16, 4, 128
    q, k, v = _decode_inputs(B, 1, Lk, Hq, Hkv, D, D, torch.bfloat16, cuda_device)
    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        for _ in range(2):
            xattn.causal_flash_attn_fwd(q, k, v)
    torch.cuda.current_stream(cuda_device).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y, lse = xattn.causal_flash_attn_fwd(q, k, v)
    for seed in (1, 2):
        q2, k2, v2 = _decode_inputs(B, 1, Lk, Hq, Hkv, D, D, torch.bfloat16, cuda_device, seed=seed)
        q.copy_(q2); k.copy_(k2); v.copy_(v2)
        graph.replay()
        y_eager, lse_eager = xattn.causal_flash_attn_fwd(q2, k2, v2)
        assert torch.equal(y, y_eager) and torch.equal(lse, lse_eager)
    xattn.check_status()
