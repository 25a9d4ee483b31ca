"""GPU parity of SoftDelta attention (causal, sliding-window, sliding-chunk) against the CPU oracle.
Structure and bounds follow the reference's SoftDelta tests
(tests/softdelta/test_softdelta_attention.py:58-145): the output error is bounded by the composed
tolerance of the two reads and the gate, gradients by the element-wise tolerances plus a relative-norm
bound (5e-3 fp16, 3e-2 bf16)."""
import pytest
import torch
import torch.nn.functional as F

import xattn_b200 as xattn
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

GRAD_REL_NORM = {torch.float16: 5e-3, torch.bfloat16: 3e-2}
HEADS = ((4, 4), (4, 2), (4, 1), (12, 3))
CASES = {
    "length-one": dict(length=1),
    "length-two": dict(length=2),
    "uneven": dict(length=17),
    "block-boundary": dict(length=129),
    "segments": dict(length=150, segments=(1, 2, 40, 3, 64, 7)),
    "bos": dict(length=150, bos=(5, 1, 70, 2)),
}


def make_inputs(dev, dtype, batch, length, q_heads, kv_heads, dim, vdim, with_k_read, q_length=None, prev=0, seed=0):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    q_length = length if q_length is None else q_length
    r = lambda *s: torch.randn(s, generator=gen).to(device=dev, dtype=dtype)
    t = dict(
        q=F.normalize(r(batch, q_length, q_heads, dim), dim=-1),
        k=F.normalize(r(batch, length, kv_heads, dim), dim=-1),
        v=F.silu(r(batch, length, kv_heads, vdim)) + 0.1,
        g=r(batch, q_length, q_heads) * 0.75,
        k_read=F.normalize(F.silu(r(batch, q_length, kv_heads, dim)), dim=-1) if with_k_read else None,
        prev_k=None, prev_v=None,
    )
    if prev:
        t["prev_k"] = F.normalize(r(batch, prev, kv_heads, dim), dim=-1)
        t["prev_v"] = F.silu(r(batch, prev, kv_heads, vdim)) + 0.1
    return t


def run_lengths(batch, length, lengths, dev):
    rows = []
    for b in range(batch):
        ids, sid, i = [], 0, b
        while len(ids) < length:
            ids += [sid] * lengths[i % len(lengths)]
            sid += 1
            i += 1
        rows.append(ids[:length])
    return torch.tensor(rows, dtype=torch.int64, device=dev)


def check(fn_name, t, dtype, level=0, op_kwargs=None, oracle_kwargs=None, metadata=None):
    op_kwargs, oracle_kwargs, metadata = op_kwargs or {}, oracle_kwargs or {}, metadata or {}
    names = [n for n in ("q", "k", "v", "g", "k_read", "prev_k", "prev_v") if t[n] is not None]
    leaves = {n: t[n].detach().clone().requires_grad_() for n in names}
    call = dict(q=leaves["q"], k=leaves["k"], k_read=leaves.get("k_read"), v=leaves["v"], g=leaves["g"])
    if "prev_k" in leaves:
        call.update(prev_k=leaves["prev_k"], prev_v=leaves["prev_v"])
    y = getattr(xattn, fn_name)(**call, **op_kwargs, **metadata, backend="sm90", high_precision_level=level)

    ref = {n: t[n].detach().double().cpu().requires_grad_() for n in names}
    q_ids = k_ids = None
    Lq = t["q"].shape[1]
    if "segment_idx" in metadata:
        k_ids = metadata["segment_idx"].cpu()
        q_ids = k_ids[:, -Lq:]
    if "bos_mask" in metadata:
        k_ids = metadata["bos_mask"].cumsum(1).cpu()
        q_ids = k_ids[:, -Lq:]
    expected, read, neg = O.softdelta(ref["q"], ref["k"], ref["v"], ref["g"], ref.get("k_read"),
                                      prev_k=ref.get("prev_k"), prev_v=ref.get("prev_v"),
                                      q_segment_idx=q_ids, k_segment_idx=k_ids, **oracle_kwargs)
    assert y.shape == expected.shape and y.dtype == dtype and torch.isfinite(y).all()
    rep = read.shape[2] // neg.shape[2]
    gate = torch.sigmoid(ref["g"].detach())[..., None]
    a, r_ = O.ATOL[dtype], O.RTOL[dtype]
    bound = (a + r_ * read.abs() + gate * (a + r_ * neg.repeat_interleave(rep, 2).abs()) + a + r_ * expected.abs()).detach()
    err = (y.detach().double().cpu() - expected.detach()).abs()
    assert bool((err <= bound).all()), f"composed error ratio {(err / bound).max().item()}"

    gen = torch.Generator(device="cpu").manual_seed(7)
    dy = (torch.randn(y.shape, generator=gen) / y.numel() ** 0.5).to(device=y.device, dtype=dtype)
    grads = torch.autograd.grad(y, list(leaves.values()), dy, retain_graph=True)
    expected_grads = torch.autograd.grad(expected, list(ref.values()), dy.double().cpu())
    for name, g_, e in zip(names, grads, expected_grads):
        assert g_.dtype == dtype and g_.shape == e.shape, name
        torch.testing.assert_close(g_.cpu(), e.to(dtype), rtol=O.RTOL[dtype], atol=O.GRAD_ATOL[dtype],
                                   msg=lambda m: f"{name}: {m}")
        floor = O.GRAD_ATOL[dtype] * e.numel() ** 0.5
        rel = ((g_.double().cpu() - e).norm() / e.norm().clamp_min(floor)).item()
        assert rel < GRAD_REL_NORM[dtype], f"{name}: relative norm error {rel}"
    again = torch.autograd.grad(y, list(leaves.values()), dy)
    for g1, g2 in zip(grads, again):
        assert torch.equal(g1, g2)
    return y, grads, call, dy


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("heads", HEADS, ids=[f"h{h}kv{k}" for h, k in HEADS])
@pytest.mark.parametrize("with_k_read", (False, True), ids=("neg-key", "neg-given"))
@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16), ids=("fp16", "bf16"))
@pytest.mark.parametrize("level", (0, 1))
def test_causal_matches_oracle(case, heads, with_k_read, dtype, level, cuda_device):
    spec = CASES[case]
    t = make_inputs(cuda_device, dtype, 2, spec["length"], heads[0], heads[1], 64, 64, with_k_read, seed=20261020)
    metadata = {}
    if "segments" in spec:
        metadata["segment_idx"] = run_lengths(2, spec["length"], spec["segments"], cuda_device)
    if "bos" in spec:
        ids = run_lengths(2, spec["length"], spec["bos"], cuda_device)
        bos = torch.ones_like(ids, dtype=torch.bool)
        bos[:, 1:] = ids[:, 1:] != ids[:, :-1]
        metadata["bos_mask"] = bos
    check("softdelta_attention", t, dtype, level, metadata=metadata)


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16), ids=("fp16", "bf16"))
@pytest.mark.parametrize("with_k_read", (False, True), ids=("neg-key", "neg-given"))
@pytest.mark.parametrize("variant", ("window", "window-short-q", "chunk", "chunk-prev", "chunk-reset"))
def test_local_variants_match_oracle(variant, with_k_read, dtype, cuda_device):
    dev = cuda_device
    if variant.startswith("window"):
        q_len = 70 if variant == "window-short-q" else None
        t = make_inputs(dev, dtype, 2, 200, 4, 2, 64, 96, with_k_read, q_length=q_len, seed=3)
        check("sliding_window_softdelta_attention", t, dtype, 0, dict(window_size=33),
              dict(visibility="window", span=33),
              dict(segment_idx=run_lengths(2, 200, (60, 1, 90, 49), dev)))
    elif variant == "chunk":
        t = make_inputs(dev, dtype, 2, 200, 4, 1, 64, 64, with_k_read, seed=4)
        check("sliding_chunk_softdelta_attention", t, dtype, 0, dict(chunk_size=48), dict(visibility="chunk", span=48))
    elif variant == "chunk-prev":
        t = make_inputs(dev, dtype, 2, 130, 4, 2, 64, 64, with_k_read, prev=32, seed=5)
        check("sliding_chunk_softdelta_attention", t, dtype, 0, dict(chunk_size=32), dict(visibility="chunk", span=32))
    else:
        t = make_inputs(dev, dtype, 2, 200, 4, 2, 64, 64, with_k_read, seed=6)
        check("sliding_chunk_softdelta_attention", t, dtype, 0, dict(chunk_size=16, reset_chunk_pos_per_seq=True),
              dict(visibility="chunk", span=16, reset_position_per_segment=True),
              dict(segment_idx=run_lengths(2, 200, (60, 1, 90, 49), dev)))


def test_gqa16x4_d128_packed(cuda_device):
    t = make_inputs(cuda_device, torch.bfloat16, 1, 320, 16, 4, 128, 128, False, seed=11)
    check("softdelta_attention", t, torch.bfloat16, 0,
          metadata=dict(segment_idx=run_lengths(1, 320, (100, 1, 150, 69), cuda_device)))


@pytest.mark.parametrize("gate_value", (-30.0, 30.0))
def test_gate_extremes(gate_value, cuda_device):
    t = make_inputs(cuda_device, torch.bfloat16, 1, 65, 4, 2, 64, 64, False, seed=5)
    t["g"] = torch.full_like(t["g"], gate_value)
    check("softdelta_attention", t, torch.bfloat16)


@pytest.mark.parametrize("level", (0, 1))
def test_standalone_forward_backward(level, cuda_device):
    """_fwd returns (y, neg_read, lse) with the documented layouts; _bwd reproduces autograd's gradients."""
    dtype = torch.bfloat16
    t = make_inputs(cuda_device, dtype, 2, 150, 4, 2, 64, 64, True, seed=8)
    y, grads, call, dy = check("softdelta_attention", t, dtype, level)
    with torch.no_grad():
        args = {k: (v.detach() if v is not None else None) for k, v in call.items()}
        y2, neg_read, lse = xattn.softdelta_attention_fwd(**args, high_precision_level=level)
        assert torch.equal(y2, y.detach())
        assert neg_read.shape == (2, 150, 2, 64) and neg_read.dtype == (torch.float32 if level else dtype)
        assert lse.shape == (2, 2 + 4, 150) and lse.dtype == torch.float32
        assert torch.count_nonzero(neg_read[:, 0]) == 0          # no earlier key at position 0
        out = xattn.softdelta_attention_bwd(dy, args["q"], args["k"], args["k_read"], args["v"], args["g"],
                                            y2, neg_read, lse, high_precision_level=level)
        assert len(out) == 5
        dq, dk, dv, dg, dk_read = out
        for got, want in zip((dq, dk, dv, dg, dk_read), (grads[0], grads[1], grads[2], grads[3], grads[4])):
            assert torch.equal(got, want)


def test_k_read_none_folds_into_dk(cuda_device):
    dtype = torch.bfloat16
    t = make_inputs(cuda_device, dtype, 1, 90, 4, 2, 64, 64, False, seed=9)
    y, neg_read, lse = xattn.softdelta_attention_fwd(t["q"], t["k"], None, t["v"], t["g"])
    dy = torch.randn_like(y)
    out = xattn.softdelta_attention_bwd(dy, t["q"], t["k"], None, t["v"], t["g"], y, neg_read, lse)
    assert out[4] is None
    out2 = xattn.sliding_chunk_softdelta_attention_bwd(dy, t["q"], t["k"], None, t["v"], t["g"], y, neg_read, lse, 4096)
    assert len(out2) == 7 and out2[5] is None and out2[6] is None


# ---- value groups (the reference's internal layout: tests/softdelta/test_value_groups.py) --------
# (D, groups, group_dim): group widths of 64 channels and one that is not a multiple of 8
GROUP_DIMS = {"d128c2": (128, 2, 64), "d192c3": (192, 3, 64), "d64c4-composed": (64, 4, 12)}
GROUP_SUPPORTS = {"causal": ("full", None), "window40": ("window", 40), "chunk32": ("chunk", 32)}


@pytest.mark.parametrize("dims", list(GROUP_DIMS))
@pytest.mark.parametrize("support", list(GROUP_SUPPORTS))
@pytest.mark.parametrize("heads", ((8, 2), (16, 1)), ids=("h8kv2", "h16kv1"))
@pytest.mark.parametrize("segments", (False, True), ids=("dense", "segments"))
@pytest.mark.parametrize("with_k_read", (False, True), ids=("neg-key", "neg-given"))
@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16), ids=("fp16", "bf16"))
@pytest.mark.parametrize("level", (0, 1))
def test_value_groups_match_oracle(dims, support, heads, segments, with_k_read, dtype, level, cuda_device):
    """v [B, L, Hkv, C, Dg] with a gate per group of Dg channels (g [B, L, H, C, 1]), driven through the
    internal autograd function as the reference's own test does."""
    from xattn_b200.ops.softdelta_attention import _softdelta_value_groups
    dev = cuda_device
    qk_dim, groups, group_dim = GROUP_DIMS[dims]
    visibility, span = GROUP_SUPPORTS[support]
    batch, length = 2, 150
    gen = torch.Generator(device="cpu").manual_seed(20261025)
    r = lambda *s: torch.randn(s, generator=gen).to(device=dev, dtype=dtype)
    t = dict(
        q=F.normalize(r(batch, length, heads[0], qk_dim), dim=-1),
        k=F.normalize(r(batch, length, heads[1], qk_dim), dim=-1),
        v=F.silu(r(batch, length, heads[1], groups, group_dim)) + 0.1,
        g=r(batch, length, heads[0], groups, 1) * 0.75,
    )
    if with_k_read:
        t["k_read"] = F.normalize(F.silu(r(batch, length, heads[1], qk_dim)), dim=-1)
    ids = run_lengths(batch, length, (1, 2, 40, 3, 64, 7), dev) if segments else None
    leaves = {n: x.detach().clone().requires_grad_() for n, x in t.items()}
    y = _softdelta_value_groups(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves.get("k_read"),
                                q_segment_idx=ids, k_segment_idx=ids, visibility=visibility, span=span,
                                high_precision_level=level)
    ref = {n: x.detach().double().cpu().requires_grad_() for n, x in t.items()}
    ids_cpu = None if ids is None else ids.cpu()
    expected, read, neg = O.softdelta(ref["q"], ref["k"], ref["v"], ref["g"], ref.get("k_read"),
                                      q_segment_idx=ids_cpu, k_segment_idx=ids_cpu, visibility=visibility, span=span)
    assert y.shape == expected.shape == (batch, length, heads[0], groups, group_dim)
    assert y.dtype == dtype and torch.isfinite(y).all()
    rep = heads[0] // heads[1]
    gate = torch.sigmoid(ref["g"].detach())
    a, r_ = O.ATOL[dtype], O.RTOL[dtype]
    bound = (a + r_ * read.abs() + gate * (a + r_ * neg.repeat_interleave(rep, 2).abs()) + a + r_ * expected.abs()).detach()
    err = (y.detach().double().cpu() - expected.detach()).abs()
    assert bool((err <= bound).all()), f"composed error ratio {(err / bound).max().item()}"
    dy = (torch.randn(y.shape, generator=gen) / y.numel() ** 0.5).to(device=dev, dtype=dtype)
    grads = torch.autograd.grad(y, list(leaves.values()), dy)
    expected_grads = torch.autograd.grad(expected, list(ref.values()), dy.double().cpu())
    for name, g_, e in zip(leaves, grads, expected_grads):
        assert g_.dtype == dtype and g_.shape == e.shape, name
        torch.testing.assert_close(g_.cpu(), e.to(dtype), rtol=O.RTOL[dtype], atol=O.GRAD_ATOL[dtype],
                                   msg=lambda m: f"{name}: {m}")
        floor = O.GRAD_ATOL[dtype] * e.numel() ** 0.5
        rel = ((g_.double().cpu() - e).norm() / e.norm().clamp_min(floor)).item()
        assert rel < GRAD_REL_NORM[dtype], f"{name}: relative norm error {rel}"


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16), ids=("fp16", "bf16"))
@pytest.mark.parametrize("shape,tail_len", (((2, 300, 2, 64), 0), ((3, 257, 1, 96), 100), ((1, 4099, 4, 128), 4099),
                                            ((2, 5, 3, 8), 1)))
def test_merge_gradients_is_an_fp32_sum_rounded_once(shape, tail_len, dtype, cuda_device):
    """out = a + b (+ tail on the last rows of each batch row), bit for bit the FP32 sum rounded to the dtype
    (the role of _softdelta_merge_gradients, xattn/ops/softdelta_attention.py:506-516)."""
    from xattn_b200 import _native
    gen = torch.Generator(device="cpu").manual_seed(17)
    a = torch.randn(shape, generator=gen).to(device=cuda_device, dtype=dtype)
    b = (torch.randn(shape, generator=gen) * 3).to(device=cuda_device, dtype=dtype)
    tail = None
    expected = a.float() + b.float()
    if tail_len:
        tail = torch.randn((shape[0], tail_len, *shape[2:]), generator=gen).to(device=cuda_device, dtype=dtype)
        expected[:, shape[1] - tail_len:] += tail.float()
    out = _native.softdelta_merge_gradients(a, b, tail)
    assert out.dtype == dtype and torch.equal(out, expected.to(dtype))
