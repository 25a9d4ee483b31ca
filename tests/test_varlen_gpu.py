"""Packed variable-length inputs, following the reference's check_packed (tests/_numerics.py:238-272):
sequences of length 0 / 1 / 17 / 65 against K sequences 0 / 5 / 41 / 129, right-aligned pairing."""
import pytest
import torch
import torch.nn.functional as F

from oracle import attention_oracle as O
from xattn_b200.ops.sliding_chunk_attention import _flash_sca_varlen
from xattn_b200.ops.sliding_window_attention import _flash_swa_varlen

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("operation", ("window", "chunk"))
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16), ids=("bf16", "fp16"))
@pytest.mark.parametrize("kv_heads", (1, 4))
def test_packed(operation, dtype, kv_heads, cuda_device):
    torch.manual_seed(513)
    dev = cuda_device
    q_lengths, k_lengths = (0, 1, 17, 65), (0, 5, 41, 129)
    q = F.normalize(torch.randn(sum(q_lengths), 4, 64, device=dev, dtype=dtype), dim=-1).requires_grad_()
    k = F.normalize(torch.randn(sum(k_lengths), kv_heads, 64, device=dev, dtype=dtype), dim=-1).requires_grad_()
    v = (F.silu(torch.randn(sum(k_lengths), kv_heads, 96, device=dev, dtype=dtype)) + 0.1).requires_grad_()
    cu_q = torch.tensor((0, *torch.tensor(q_lengths).cumsum(0).tolist()), device=dev, dtype=torch.int32)
    cu_k = torch.tensor((0, *torch.tensor(k_lengths).cumsum(0).tolist()), device=dev, dtype=torch.int32)
    refs = [t.detach().double().cpu().requires_grad_() for t in (q, k, v)]
    parts, qs, ks = [], 0, 0
    for lq, lk in zip(q_lengths, k_lengths):
        if lq:
            mask, _ = O.allowed_masks(lq, lk, 1, operation, 32)
            parts.append(O.attention_from_mask(refs[0][None, qs:qs + lq], refs[1][None, ks:ks + lk],
                                               refs[2][None, ks:ks + lk], mask, 64 ** -0.5).squeeze(0))
        qs += lq
        ks += lk
    expected = torch.cat(parts)
    options = dict(cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=max(q_lengths), max_seqlen_k=max(k_lengths))
    if operation == "chunk":
        actual = _flash_sca_varlen(q, k, v, 32, reset_chunk_pos_per_seq=True, **options)
    else:
        actual = _flash_swa_varlen(q, k, v, 32, **options)
    torch.testing.assert_close(actual.cpu(), expected.detach().to(dtype), atol=O.ATOL[dtype], rtol=O.RTOL[dtype])
    dy = torch.randn_like(actual) / actual.numel() ** 0.5
    reference = torch.autograd.grad(expected, refs, dy.double().cpu())
    grads = torch.autograd.grad(actual, (q, k, v), dy, retain_graph=True)
    for g, r in zip(grads, reference):
        torch.testing.assert_close(g.cpu(), r.to(dtype), atol=O.GRAD_ATOL[dtype], rtol=O.RTOL[dtype])
    for a, b in zip(grads, torch.autograd.grad(actual, (q, k, v), dy)):
        assert torch.equal(a, b)
