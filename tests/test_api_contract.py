"""Argument validation of the public ops, runnable without a GPU.  Follows the reference's API
contract tests (tests/test_high_precision.py:37-86): bad levels, non-finite scales and bad head
dimensions are rejected before any tensor is read."""
import inspect

import pytest
import torch

import xattn_b200 as xattn

FAMILIES = ("causal_flash_attn", "flash_sca", "flash_swa", "softdelta_attention",
            "sliding_chunk_softdelta_attention", "sliding_window_softdelta_attention")
ENTRIES = [getattr(xattn, name + suffix) for name in FAMILIES for suffix in ("", "_fwd", "_bwd")]
INVALID_LEVELS = ((-1, ValueError), (2, ValueError), (100, ValueError), (False, TypeError), (True, TypeError),
                  (1.0, TypeError), ("1", TypeError), (None, TypeError))


def _required(fn):
    return {n: None for n, p in inspect.signature(fn).parameters.items() if p.default is inspect.Parameter.empty}


def test_public_names_match_reference():
    expected = {f + s for f in FAMILIES for s in ("", "_fwd", "_bwd")} | {"flash_sca_sm90_available"}
    assert expected <= set(xattn.__all__)


@pytest.mark.parametrize("fn", ENTRIES, ids=lambda f: f.__name__)
@pytest.mark.parametrize("value,error", INVALID_LEVELS)
def test_invalid_level_rejected_before_tensor_access(fn, value, error):
    kwargs = _required(fn)
    kwargs["high_precision_level"] = value
    with pytest.raises(error, match="high_precision_level"):
        fn(**kwargs)


@pytest.mark.parametrize("fn", ENTRIES, ids=lambda f: f.__name__)
@pytest.mark.parametrize("scale", (float("inf"), float("-inf"), float("nan")))
def test_nonfinite_scale_rejected(fn, scale):
    kwargs = _required(fn)
    kwargs["scale"] = scale
    with pytest.raises(ValueError, match="scale must be finite"):
        fn(**kwargs)


def test_window_and_chunk_arguments():
    q = torch.zeros(1, 4, 2, 8, dtype=torch.bfloat16)
    with pytest.raises(TypeError, match="window_size"):
        xattn.flash_swa(q, q, q, window_size=True)
    with pytest.raises(ValueError, match="nonnegative"):
        xattn.flash_swa(q, q, q, window_size=-1)
    with pytest.raises(ValueError, match="positive"):
        xattn.flash_sca(q, q, q, chunk_size=0)
    with pytest.raises(NotImplementedError, match="sda"):
        xattn.flash_sca(q, q, q, chunk_size=4, attn_method="sda")
    with pytest.raises(ValueError, match="attn_method"):
        xattn.flash_sca(q, q, q, chunk_size=4, attn_method="other")


def test_input_validation_messages():
    q = torch.zeros(1, 4, 2, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="4D"):
        xattn.causal_flash_attn(q[0], q, q)
    with pytest.raises(ValueError, match="share a dtype"):
        xattn.causal_flash_attn(q, q.half(), q)
    with pytest.raises(ValueError, match="fp16 and bf16"):
        xattn.causal_flash_attn(q.float(), q.float(), q.float())
    with pytest.raises(ValueError, match="q length"):
        xattn.causal_flash_attn(torch.zeros(1, 5, 2, 8, dtype=torch.bfloat16), q, q)
    with pytest.raises(ValueError, match="divisible"):
        xattn.causal_flash_attn(torch.zeros(1, 4, 3, 8, dtype=torch.bfloat16), q, q)
    with pytest.raises(ValueError, match="provided together"):
        xattn.flash_swa(q, q, q, 2, prev_k=q)
    with pytest.raises(ValueError, match="chunk_size"):
        xattn.flash_sca(q, q, q, chunk_size=3, prev_k=q, prev_v=q)
    with pytest.raises(ValueError, match="backend"):
        xattn.causal_flash_attn(q, q, q, backend="tpu")
    # no CPU path
    with pytest.raises(RuntimeError, match="CUDA"):
        xattn.causal_flash_attn(q, q, q)


def test_segment_metadata_validation():
    from xattn_b200.ops._validation import resolve_segments
    q = torch.zeros(2, 3, 1, 8)
    ids = torch.zeros(2, 5, dtype=torch.int64)
    qi, ki = resolve_segments(q, 5, ids, None, None, None, api_name="t")
    assert qi.shape == (2, 3) and ki.shape == (2, 5)
    bos = torch.zeros(2, 5, dtype=torch.bool)
    bos[:, 0] = True
    bos[0, 3] = True
    qi, ki = resolve_segments(q, 5, None, None, None, bos, api_name="t")
    assert ki[0].tolist() == [1, 1, 1, 2, 2] and qi[0].tolist() == [1, 2, 2]
    with pytest.raises(ValueError, match="mutually exclusive"):
        resolve_segments(q, 5, ids, None, None, bos, api_name="t")
    with pytest.raises(ValueError, match="provided together"):
        resolve_segments(q, 5, None, ids[:, :3], None, None, api_name="t")
    with pytest.raises(ValueError, match="int64"):
        resolve_segments(q, 5, None, ids[:, :3].int(), ids, None, api_name="t")
    with pytest.raises(ValueError, match="shape"):
        resolve_segments(q, 5, ids[:, :4], None, None, None, api_name="t")


def test_softdelta_torch_plan_matches_oracle_on_cpu():
    """backend='torch' is the reference's CPU-runnable correctness plan
    (tests/softdelta/test_softdelta_attention.py:178-184)."""
    from oracle import attention_oracle as O
    torch.manual_seed(3)
    q = torch.randn(2, 9, 4, 16).bfloat16()
    k = torch.randn(2, 12, 2, 16).bfloat16()
    v = torch.randn(2, 12, 2, 8).bfloat16()
    g = torch.randn(2, 9, 4).bfloat16()
    for name, kw, okw in (
        ("softdelta_attention", {}, {}),
        ("sliding_window_softdelta_attention", dict(window_size=3), dict(visibility="window", span=3)),
        ("sliding_chunk_softdelta_attention", dict(chunk_size=4), dict(visibility="chunk", span=4)),
    ):
        y = getattr(xattn, name)(q, k, None, v, g, backend="torch", **kw)
        ref, _, _ = O.softdelta(q.double(), k.double(), v.double(), g.double(), None, **okw)
        assert y.dtype == torch.bfloat16 and y.shape == ref.shape
        torch.testing.assert_close(y.double(), ref, atol=2e-2, rtol=2e-2)


def test_value_group_entry_checks_layout():
    """The internal value-group entry wants v [B, L, Hkv, C, Dg] and g [B, Lq, H, C, 1]
    (tests/softdelta/test_value_groups.py:1-7); other layouts are refused before any kernel runs."""
    import torch
    from xattn_b200.ops.softdelta_attention import _softdelta_value_groups
    q = torch.zeros(1, 4, 2, 8)
    k = torch.zeros(1, 4, 1, 8)
    with pytest.raises(ValueError, match="5D"):
        _softdelta_value_groups(q, k, torch.zeros(1, 4, 1, 16), torch.zeros(1, 4, 2))
    with pytest.raises(ValueError, match=r"\[B, Lq, H, C, 1\]"):
        _softdelta_value_groups(q, k, torch.zeros(1, 4, 1, 2, 8), torch.zeros(1, 4, 2, 3, 1))


def test_bench_window_slices_balance_the_work():
    """bench.py cuts the sharded window workload into slices of equal work where every slice can hold a window."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    S, window = 32768, 4096
    assert bench.window_slice_bounds(S, 1, window) == [0, S]
    assert bench.window_slice_bounds(S, 2, window) == [0, 17408, S]
    assert bench.window_slice_bounds(S, 4, window) == [0, 9728, 17408, 25088, S]
    assert bench.window_slice_bounds(S, 8, window) == [r * 4096 for r in range(9)]          # a slice is one window
    assert bench.window_slice_bounds(S, 4, window, equal=True) == [r * 8192 for r in range(5)]
    short = bench.window_slice_bounds(S, 8, window, shortest=window // 2)
    assert [b - a for a, b in zip(short, short[1:])] == [5888] + [3840] * 7
    work = lambda a, b: sum(min(i, window) + 1 for i in range(a, b))
    for world in (2, 4):
        bounds = bench.window_slice_bounds(S, world, window)
        shares = [work(a, b) for a, b in zip(bounds, bounds[1:])]
        assert max(shares) / (sum(shares) / world) < 1.01
