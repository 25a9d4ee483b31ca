"""GPU parity of causal / sliding-window / sliding-chunk attention against the CPU oracle, through
the public ops (and so through the C ABI).  Structure and tolerances follow the reference's
check_case (tests/_numerics.py:185-213): output and gradients within ATOL / GRAD_ATOL + RTOL*|ref|
of the FP64 oracle evaluated on the already-rounded inputs, standalone _fwd / _bwd, inference
mode, and bitwise-repeatable gradients."""
import pytest
import torch

import xattn_b200 as xattn
from oracle import attention_oracle as O
from tests._cases import Case, cases_for, make_inputs, metadata_for, op_options

pytestmark = pytest.mark.gpu

OPS = {"full": "causal_flash_attn", "window": "flash_swa", "chunk": "flash_sca"}
DTYPES = (torch.bfloat16, torch.float16)


def oracle_outputs(operation, case, inputs, qi, ki, dy):
    refs = [t.detach().double().cpu().requires_grad_() for t in inputs]
    q, k, v = refs[:3]
    if case.previous:
        k, v = torch.cat((refs[-2], k), 1), torch.cat((refs[-1], v), 1)
    cpu = lambda t: None if t is None else t.cpu()
    inc, _ = O.allowed_masks(case.q_length, k.shape[1], case.batch, operation, case.span, cpu(qi), cpu(ki), case.reset)
    y = O.attention_from_mask(q, k, v, inc, case.dim ** -0.5)
    grads = torch.autograd.grad(y, refs, dy.double().cpu())
    return y.detach(), grads


def assert_output(actual, expected, dtype):
    assert actual.dtype == dtype and actual.shape == expected.shape
    assert torch.isfinite(actual).all()
    torch.testing.assert_close(actual.cpu(), expected.to(dtype), atol=O.ATOL[dtype], rtol=O.RTOL[dtype])


def assert_grads(actual, expected, dtype):
    assert len(actual) == len(expected)
    for g, r in zip(actual, expected):
        assert g is not None and torch.isfinite(g).all()
        torch.testing.assert_close(g.cpu(), r.to(dtype), atol=O.GRAD_ATOL[dtype], rtol=O.RTOL[dtype])


def check_case(operation, case, dtype, kv_heads, level, device, deterministic=True):
    inputs = make_inputs(operation, case, dtype, kv_heads, device)
    meta, qi, ki = metadata_for(case, device)
    options = {**op_options(operation, case, inputs), **meta, "backend": "sm90"}
    fn = getattr(xattn, OPS[operation])
    base = inputs[:3]
    y = fn(*base, **options, deterministic=deterministic, high_precision_level=level)
    gen = torch.Generator(device="cpu").manual_seed(11)
    dy = (torch.randn(y.shape, generator=gen) / y.numel() ** 0.5).to(device=device, dtype=dtype)
    expected, expected_grads = oracle_outputs(operation, case, inputs, qi, ki, dy)
    assert_output(y, expected, dtype)
    grads = torch.autograd.grad(y, inputs, dy, retain_graph=True)
    assert_grads(grads, expected_grads, dtype)
    again = torch.autograd.grad(y, inputs, dy)
    for a, b in zip(grads, again):
        assert torch.equal(a, b), "gradients must be bitwise repeatable"
    fwd, bwd = getattr(xattn, OPS[operation] + "_fwd"), getattr(xattn, OPS[operation] + "_bwd")
    with torch.no_grad():
        y2, lse = fwd(*base, **options, high_precision_level=level)
        assert_output(y2, expected, dtype)
        assert lse.dtype == torch.float32 and lse.shape == (case.batch, 4, case.q_length)
        g2 = bwd(dy, *base, y2, lse, **options, deterministic=deterministic, high_precision_level=level)
        assert_grads([g for g in g2[:len(inputs)]], expected_grads, dtype)
    with torch.inference_mode():
        assert_output(fn(*base, **options, high_precision_level=level), expected, dtype)


def _params():
    out = []
    for operation in OPS:
        for case in cases_for(operation):
            out.append(pytest.param(operation, case, id=f"{operation}-{case.name}"))
    return out


@pytest.mark.parametrize("operation,case", _params())
@pytest.mark.parametrize("dtype", DTYPES, ids=("bf16", "fp16"))
@pytest.mark.parametrize("kv_heads", (1, 2, 4), ids=("mqa", "gqa", "mha"))
def test_case_level0(operation, case, dtype, kv_heads, cuda_device):
    check_case(operation, case, dtype, kv_heads, 0, cuda_device)


@pytest.mark.parametrize("operation,case", _params())
@pytest.mark.parametrize("dtype", DTYPES, ids=("bf16", "fp16"))
def test_case_level1(operation, case, dtype, cuda_device):
    check_case(operation, case, dtype, 2, 1, cuda_device)


@pytest.mark.parametrize("operation", OPS)
@pytest.mark.parametrize("length", (7, 193, 513))
@pytest.mark.parametrize("dim,value_dim", ((32, 32), (64, 128), (96, 64), (128, 128), (160, 96), (192, 192), (256, 256)))
def test_head_dimension_buckets(operation, length, dim, value_dim, cuda_device):
    case = Case("dims", length, length, dim, value_dim, span=3 if length == 7 else 255, batch=1)
    check_case(operation, case, torch.bfloat16, 2, 0, cuda_device)


def test_lse_and_empty_rows(cuda_device):
    """Rows without a visible key: y = 0, lse = -inf, zero gradients; other rows' lse matches."""
    case = Case("empty", 17, 41, 64, 64, metadata="unmatched")
    inputs = make_inputs("full", case, torch.bfloat16, 2, cuda_device)
    meta, qi, ki = metadata_for(case, cuda_device)
    y, lse = xattn.causal_flash_attn_fwd(*inputs, **meta)
    assert torch.count_nonzero(y) == 0 and torch.isinf(lse).all() and (lse < 0).all()
    case = Case("lse", 129, 257, 64, 64, metadata="independent")
    inputs = make_inputs("full", case, torch.bfloat16, 2, cuda_device)
    meta, qi, ki = metadata_for(case, cuda_device)
    y, lse = xattn.causal_flash_attn_fwd(*inputs, **meta)
    inc, _ = O.allowed_masks(129, 257, 2, "full", None, qi.cpu(), ki.cpu(), False)
    ref = O.lse_from_mask(inputs[0].detach().double().cpu(), inputs[1].detach().double().cpu(), inc, 64 ** -0.5)
    finite = torch.isfinite(ref)
    torch.testing.assert_close(lse.cpu().double()[finite], ref[finite], atol=1e-4, rtol=1e-4)
    assert torch.equal(torch.isinf(lse.cpu()), ~finite)


@pytest.mark.parametrize("operation", OPS)
@pytest.mark.parametrize("scale_sign", (0, -1))
def test_nonpositive_scale(operation, scale_sign, cuda_device):
    case = Case("scale-edge", 65, 65, 64, 64, span=32, batch=1)
    dtype = torch.bfloat16
    inputs = make_inputs(operation, case, dtype, 2, cuda_device)
    options = op_options(operation, case, inputs)
    scale = scale_sign * case.dim ** -0.5
    refs = [t.detach().double().cpu().requires_grad_() for t in inputs]
    inc, _ = O.allowed_masks(65, 65, 1, operation, 32)
    expected = O.attention_from_mask(*refs, inc, scale)
    fn = OPS[operation]
    y = getattr(xattn, fn)(*inputs, **options, scale=scale)
    assert_output(y, expected.detach(), dtype)
    dy = torch.randn_like(y) / y.numel() ** 0.5
    ref_grads = torch.autograd.grad(expected, refs, dy.double().cpu())
    assert_grads(torch.autograd.grad(y, inputs, dy), ref_grads, dtype)
    y2, lse = getattr(xattn, fn + "_fwd")(*inputs, **options, scale=scale)
    grads = getattr(xattn, fn + "_bwd")(dy, *inputs, y2, lse, **options, scale=scale)[:3]
    assert_grads(grads, ref_grads, dtype)
    if scale == 0:
        assert torch.count_nonzero(grads[0]) == 0 and torch.count_nonzero(grads[1]) == 0


def test_backward_rejects_fp32_output(cuda_device):
    q = torch.zeros(1, 8, 2, 64, device=cuda_device, dtype=torch.bfloat16)
    k = v = torch.zeros(1, 8, 1, 64, device=cuda_device, dtype=torch.bfloat16)
    y = torch.zeros(1, 8, 2, 64, device=cuda_device, dtype=torch.float32)
    lse = torch.zeros(1, 2, 8, device=cuda_device)
    for name, span in (("causal_flash_attn", {}), ("flash_swa", dict(window_size=8)), ("flash_sca", dict(chunk_size=8))):
        with pytest.raises(ValueError, match="Q/K/V dtype"):
            getattr(xattn, name + "_bwd")(y.to(q.dtype), q, k, v, y, lse, **span, backend="sm90")


@pytest.mark.parametrize("dims", ((7, 16), (16, 13), (264, 16), (16, 264)))
def test_invalid_dimensions_rejected_before_launch(dims, cuda_device):
    d, w = dims
    q = torch.empty(1, 1, 1, d, device=cuda_device, dtype=torch.bfloat16)
    v = torch.empty(1, 1, 1, w, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="multiples of 8"):
        xattn.causal_flash_attn(q=q, k=None, v=v, backend="sm90")


def test_single_key_high_precision_is_exact(cuda_device):
    """With one visible key the level-1 forward returns V bit for bit
    (tests/test_high_precision.py:89-139)."""
    for dtype in DTYPES:
        q = torch.zeros(1, 1, 4, 128, device=cuda_device, dtype=dtype)
        k = torch.zeros(1, 1, 2, 128, device=cuda_device, dtype=dtype)
        q[..., 0] = 256
        k[..., 0] = 65536 if dtype == torch.bfloat16 else 4096
        v = torch.linspace(-1, 1, 256, device=cuda_device).reshape(1, 1, 2, 128).to(dtype)
        expected = v.float().repeat_interleave(2, dim=2)
        for fn, kw in ((xattn.causal_flash_attn_fwd, {}), (xattn.flash_swa_fwd, dict(window_size=256)),
                       (xattn.flash_sca_fwd, dict(chunk_size=256))):
            y, _ = fn(q, k, v, **kw, high_precision_level=1)
            assert torch.equal(y.float(), expected)


@pytest.mark.parametrize("operation", OPS)
def test_constant_key_support_level1(operation, cuda_device):
    """All visible keys identical -> dQ exactly zero at level 1 (tests/test_high_precision.py:247-275)."""
    n, d = 384, 64
    dtype = torch.bfloat16
    q = torch.zeros(1, n, 4, d, device=cuda_device, dtype=dtype)
    q[..., 0] = 1
    k = torch.zeros(1, n, 2, d, device=cuda_device, dtype=dtype)
    if operation == "full":
        k[..., 0] = 800
        start = 0
    else:
        k[:, 0, :, 0] = 800
        start = 256
    v = torch.randn(1, n, 2, d, device=cuda_device).to(dtype)
    for t in (q, k, v):
        t.requires_grad_()
    options = dict(high_precision_level=1)
    if operation == "chunk":
        options["chunk_size"] = 128
    elif operation == "window":
        options["window_size"] = 127
    out = getattr(xattn, OPS[operation])(q, k, v, **options)
    grads = torch.autograd.grad(out, (q, k, v), torch.ones_like(out))
    assert all(torch.isfinite(g).all() for g in grads)
    assert torch.count_nonzero(grads[0][:, start:]) == 0


def test_long_sequence_properties(cuda_device):
    """Headline shape, size-independent checks: sampled rows against the oracle, segment isolation
    (a packed row equals its segments run alone: bit for bit when the segment starts on a tile-pair
    boundary, so that both runs tile it identically; within rounding otherwise), and bitwise
    repeatability."""
    torch.manual_seed(5)
    B, S, Hq, Hkv, D = 1, 8192, 8, 2, 128
    q = torch.randn(B, S, Hq, D, device=cuda_device, dtype=torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device=cuda_device, dtype=torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, device=cuda_device, dtype=torch.bfloat16)
    bounds = [0, 1536, 4096, 5000, 8192]
    ids = torch.zeros(B, S, dtype=torch.int64, device=cuda_device)
    for i in range(len(bounds) - 1):
        ids[:, bounds[i]:bounds[i + 1]] = i
    y, lse = xattn.causal_flash_attn_fwd(q, k, v, segment_idx=ids)
    dy = torch.randn_like(y)
    dq, dk, dv = xattn.causal_flash_attn_bwd(dy, q, k, v, y, lse, segment_idx=ids)
    for i in range(len(bounds) - 1):
        a, b = bounds[i], bounds[i + 1]
        ys, ls = xattn.causal_flash_attn_fwd(q[:, a:b], k[:, a:b], v[:, a:b])
        gq, gk, gv = xattn.causal_flash_attn_bwd(dy[:, a:b], q[:, a:b], k[:, a:b], v[:, a:b], ys, ls)
        pairs = ((ys, y[:, a:b]), (ls, lse[:, :, a:b]), (gq, dq[:, a:b]), (gk, dk[:, a:b]), (gv, dv[:, a:b]))
        for alone, packed in pairs:
            if a % 256 == 0:
                assert torch.equal(alone, packed)
            else:
                torch.testing.assert_close(alone.float(), packed.float(), atol=2e-2, rtol=2e-2)
    rows = torch.tensor([0, 1, 127, 128, 1535, 1536, 4095, 4096, 8191])
    qd, kd, vd = q.double().cpu(), k.double().cpu(), v.double().cpu()
    inc, _ = O.allowed_masks(S, S, B, "full", None, ids.cpu(), ids.cpu(), False)
    ref = O.attention_from_mask(qd[:, rows], kd, vd, inc[:, rows], D ** -0.5)
    torch.testing.assert_close(y[:, rows].cpu(), ref.to(torch.bfloat16), atol=1e-2, rtol=1e-2)
    dq2, dk2, dv2 = xattn.causal_flash_attn_bwd(dy, q, k, v, y, lse, segment_idx=ids)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
    # the warp roles of the kernels hand tiles to each other through barriers: a slip there shows as
    # a run that differs, so repeat the dense form of the shape a few times
    yd, lsed = xattn.causal_flash_attn_fwd(q, k, v)
    gd = xattn.causal_flash_attn_bwd(dy, q, k, v, yd, lsed)
    for _ in range(4):
        y2, lse2 = xattn.causal_flash_attn_fwd(q, k, v)
        assert torch.equal(yd, y2) and torch.equal(lsed, lse2)
        for a, b in zip(gd, xattn.causal_flash_attn_bwd(dy, q, k, v, yd, lsed)):
            assert torch.equal(a, b)
