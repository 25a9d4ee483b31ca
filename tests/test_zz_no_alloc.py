"""The allocation-free backward entry point (xattn_b200_bwd_static_scratch).

It exists for callers that are not allowed to allocate device memory — an application that owns
the whole device arena and gives an op only its input and output buffers, or a serving loop that
cannot take the device-wide stall of a cudaMalloc — so its scratch is a fixed array inside the
library.  The test calls it through the C ABI twice in a row (the second time on a different,
smaller problem, so that whatever the first call left in the shared array would show up if it were
ever read) and compares with the regular entry point, which takes a caller-allocated workspace.
The kernels are deterministic, so the results must be equal bit for bit.  The file name keeps this
test last in collection order."""
import ctypes as C

import pytest
import torch

from xattn_b200 import _lib, _native


@pytest.mark.gpu
def test_static_scratch_backward_matches_regular_entry(cuda_device):
    dev = cuda_device
    torch.manual_seed(1234)
    for B, Lq, Lk, Hq, Hkv, D, V, window in ((2, 300, 428, 4, 2, 128, 128, 77), (1, 65, 65, 4, 4, 64, 96, None)):
        dtype = torch.bfloat16
        q = torch.randn(B, Lq, Hq, D, device=dev, dtype=dtype)
        k = torch.randn(B, Lk, Hkv, D, device=dev, dtype=dtype)
        v = torch.randn(B, Lk, Hkv, V, device=dev, dtype=dtype)
        kw = dict(visibility="full") if window is None else dict(visibility="window", span=window)
        plan = _native.build_plan(B, Lq, Lk, dev, **kw)
        scale = D ** -0.5
        y, lse = _native.attention_fwd(q, k, v, plan, scale)
        dy = torch.randn_like(y)
        want = _native.attention_bwd(dy, q, k, v, y, lse, plan, scale)
        # outputs exist before the call; poison them so that an entry point that did nothing is caught
        got = [torch.full_like(t, float("nan")) for t in want]
        _native.prepare_device(dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        _native.attention_bwd_static_scratch(dy, q, k, v, y, lse, plan, scale, *got)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before, "the entry point must not allocate through torch"
        # a raw cudaMalloc would not show in torch's counter: the driver's free-memory figure must not
        # move either across a further call (the first one may have loaded the module)
        free_before = torch.cuda.mem_get_info(dev)[0]
        again = [torch.empty_like(t) for t in want]
        torch.cuda.synchronize()
        free_mid = torch.cuda.mem_get_info(dev)[0]        # after torch took what `again` needs
        _native.attention_bwd_static_scratch(dy, q, k, v, y, lse, plan, scale, *again)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_mid <= free_before, "device memory was taken during the call"
        for a, b in zip(again, want):
            assert torch.equal(a, b)
        _native.check_status()
        for name, a, b in zip(("dq", "dk", "dv"), got, want):
            assert torch.isfinite(a).all(), name
            assert torch.equal(a, b), f"{name} differs from the regular entry point"


@pytest.mark.gpu
def test_static_scratch_rejects_oversized_problems(cuda_device):
    lib = _lib.load()
    args = _lib.BwdArgs()
    args.dtype = _lib.XATTN_DTYPE_BF16
    args.batch, args.q_heads, args.q_len = 8, 32, 8192        # 2 Mi rows > 1 Mi
    args.k_len, args.kv_heads, args.qk_dim, args.v_dim = 8192, 8, 128, 128
    rc = lib.xattn_b200_bwd_static_scratch(C.byref(args), None)
    assert rc == -1
    assert "exceeds the static workspace" in _lib.last_error()


def test_static_scratch_symbol_is_exported():
    lib = _lib.load()
    assert hasattr(lib, "xattn_b200_bwd_static_scratch")
    assert _native.STATIC_SCRATCH_MAX_ROWS == 1 << 20
