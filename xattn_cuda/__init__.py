"""``xattn_cuda``: the native-op module the reference's Python layer imports, over libxattn_b200.

The reference builds this module from csrc/xattn_extension.cc:9-20 (pybind, torch tensors in and out)
and its L4 reaches every kernel through ``xattn_cuda.ops.<name>`` obtained lazily
(xattn/ops/_causal_attention.py:36-45).  Here the same names are thin torch-facing functions over the
C ABI of include/xattn_b200.h: they allocate the outputs, build the mask plan and call
``xattn_b200_fwd`` / ``xattn_b200_bwd`` with raw pointers.  Argument order, defaults and the shape of
the returned tuples follow the pybind definitions cited at each function.

Provided: the causal / sliding-window / sliding-chunk forward and backward ops with their component,
strict-past and packed-varlen forms, BOS-mask helpers, and the SoftDelta gate / merge ops.  Not
provided, because this library does the same work differently and the names would have nothing to
bind to: the packed-route planners of the sliding-chunk op (``_flash_sca_sm90_bos_plan``,
``_paired_bos_plan``, ``*_metadata_is_dense``, ``_build_row_aligned_metadata``, the try / store entries
of the inference plan cache, whose role the transparent plan cache of ``xattn_b200.ops._core`` plays)
— a BOS mask becomes segment ids and one kernel family serves every packing; the fused
``_softdelta_fwd`` / ``_softdelta_bwd`` launches; and the eleven ``_attention_precision_*`` stages —
level 1 is the anchored backward inside ``xattn_b200_bwd`` (``high_precision=True`` on the backward
ops below selects it).  ``backend`` accepts the reference's spellings and selects the only backend
there is.  There is no CPU path: without the built library every op raises.
"""
from __future__ import annotations

import types
from typing import Optional

import torch

from xattn_b200 import _native
from xattn_b200.ops import _core, _varlen
from xattn_b200.ops._validation import normalize_backend

ops = types.ModuleType("xattn_cuda.ops", "Native attention ops (sm_100a) under the reference's op names.")

Support = _core.Support


def _export(fn):
    setattr(ops, fn.__name__, fn)
    return fn


def _fwd(q, k, v, support, scale, prev_k, prev_v, q_seg, k_seg, backend, output_state, high_precision):
    normalize_backend(backend, "xattn_cuda")
    return _core.forward(q, k, v, support, float(scale), prev_k, prev_v, q_seg, k_seg,
                         high_precision=bool(high_precision), output_state=output_state)


def _bwd(dy, q, k, v, y, lse, support, scale, prev_k, prev_v, q_seg, k_seg, backend, fp32_kv_grads=False,
         high_precision=False):
    normalize_backend(backend, "xattn_cuda")
    dq, dk, dv, dpk, dpv = _core.backward(dy, q, k, v, y, lse, support, float(scale), prev_k, prev_v, q_seg, k_seg,
                                          high_precision=bool(high_precision))
    if fp32_kv_grads:
        # the reference hands back its FP32 accumulators; dK / dV never leave the tensor memory
        # unrounded here, so these are the rounded values widened
        dk, dv = dk.float(), dv.float()
        dpk, dpv = (None if t is None else t.float() for t in (dpk, dpv))
    return dq, dk, dv, dpk, dpv


# ---- causal (csrc/causal_flash_attn/causal_flash_attn.cc:78-122) ---------------------------------

@_export
def causal_flash_attn_fwd(q, k, v, scale, q_segment_idx=None, k_segment_idx=None, backend="auto",
                          output_state=None, use_fast_reciprocal=True, high_precision=False):
    """(y, lse)."""
    return _fwd(q, k, v, Support("full"), scale, None, None, q_segment_idx, k_segment_idx, backend, output_state,
                high_precision)


@_export
def causal_flash_attn_bwd(y_grad, q, k, v, y, lse, scale, q_segment_idx=None, k_segment_idx=None,
                          deterministic=False, backend="auto", high_precision=False):
    """(dq, dk, dv)."""
    return _bwd(y_grad, q, k, v, y, lse, Support("full"), scale, None, None, q_segment_idx, k_segment_idx, backend,
                high_precision=high_precision)[:3]


@_export
def _causal_flash_attn_component_fwd(q, k, v, scale, prev_k=None, prev_v=None, q_segment_idx=None,
                                     k_segment_idx=None, backend="auto", output_state=None, strict_past=False,
                                     use_fast_reciprocal=True, high_precision=False):
    return _fwd(q, k, v, Support("full", strict=bool(strict_past)), scale, prev_k, prev_v, q_segment_idx,
                k_segment_idx, backend, output_state, high_precision)


@_export
def _causal_flash_attn_component_bwd(y_grad, q, k, v, y, lse, scale, prev_k=None, prev_v=None, q_segment_idx=None,
                                     k_segment_idx=None, deterministic=False, backend="auto", strict_past=False,
                                     fp32_kv_grads=False, high_precision=False):
    """(dq, dk, dv, dprev_k, dprev_v)."""
    return _bwd(y_grad, q, k, v, y, lse, Support("full", strict=bool(strict_past)), scale, prev_k, prev_v,
                q_segment_idx, k_segment_idx, backend, fp32_kv_grads, high_precision)


# ---- sliding window (csrc/flash_swa/flash_swa.cc:106-178) ----------------------------------------

def _swa(window_size, strict):
    return Support("window", int(window_size), strict=strict)


@_export
def flash_swa_fwd(q, k, v, window_size, scale, prev_k=None, prev_v=None, q_segment_idx=None, k_segment_idx=None,
                  backend="auto", output_state=None, high_precision=False):
    return _fwd(q, k, v, _swa(window_size, False), scale, prev_k, prev_v, q_segment_idx, k_segment_idx, backend,
                output_state, high_precision)


@_export
def flash_swa_bwd(y_grad, q, k, v, y, lse, window_size, scale, prev_k=None, prev_v=None, q_segment_idx=None,
                  k_segment_idx=None, deterministic=False, backend="auto", fp32_kv_grads=False,
                  high_precision=False):
    return _bwd(y_grad, q, k, v, y, lse, _swa(window_size, False), scale, prev_k, prev_v, q_segment_idx,
                k_segment_idx, backend, fp32_kv_grads, high_precision)


@_export
def _flash_swa_sm90_strict_past_fwd(q, k, v, window_size, scale, prev_k=None, prev_v=None, q_segment_idx=None,
                                    k_segment_idx=None, backend="auto", output_state=None, high_precision=False):
    return _fwd(q, k, v, _swa(window_size, True), scale, prev_k, prev_v, q_segment_idx, k_segment_idx, backend,
                output_state, high_precision)


@_export
def _flash_swa_sm90_strict_past_bwd(y_grad, q, k, v, y, lse, window_size, scale, prev_k=None, prev_v=None,
                                    q_segment_idx=None, k_segment_idx=None, deterministic=False, backend="auto",
                                    high_precision=False):
    return _bwd(y_grad, q, k, v, y, lse, _swa(window_size, True), scale, prev_k, prev_v, q_segment_idx,
                k_segment_idx, backend, high_precision=high_precision)


@_export
def _flash_swa_sm90_varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, window_size, scale,
                               backend="auto", strict_past=False, output_state=None, high_precision=False):
    """Packed [T, H, D] inputs; (y [T, H, V], lse [H, T]).  A negative window is the causal form."""
    support = Support("full", strict=bool(strict_past)) if window_size < 0 else _swa(window_size, bool(strict_past))
    return _varlen.varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, support, float(scale),
                                  output_state=output_state, high_precision=bool(high_precision))


@_export
def _flash_swa_sm90_varlen_bwd(y_grad, q, k, v, y, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                               window_size, scale, deterministic=False, backend="auto", strict_past=False):
    support = Support("full", strict=bool(strict_past)) if window_size < 0 else _swa(window_size, bool(strict_past))
    return _varlen.varlen_backward(y_grad, q, k, v, y, lse, cu_seqlens_q, cu_seqlens_k, support, float(scale))


# ---- sliding chunk (csrc/flash_sca/sliding_chunk_attention.cc:674-902) ---------------------------

def _sca(chunk_size, reset, strict):
    return Support("chunk", int(chunk_size), bool(reset), strict)


@_export
def flash_sca_sm90_available(q):
    """Whether the native sliding-chunk backend can run on ``q``'s device (here: an sm_100 GPU)."""
    return bool(q.is_cuda and torch.cuda.get_device_capability(q.device)[0] == 10)


@_export
def flash_sca_fwd(q, k, v, chunk_size, scale, prev_k, prev_v, q_segment_idx, k_segment_idx, backend="auto",
                  reset_chunk_pos_per_seq=False, output_state=None, high_precision=False):
    return _fwd(q, k, v, _sca(chunk_size, reset_chunk_pos_per_seq, False), scale, prev_k, prev_v, q_segment_idx,
                k_segment_idx, backend, output_state, high_precision)


@_export
def flash_sca_bwd(y_grad, q, k, v, y, lse, chunk_size, scale, prev_k, prev_v, q_segment_idx, k_segment_idx,
                  deterministic=False, backend="auto", reset_chunk_pos_per_seq=False, fp32_kv_grads=False,
                  high_precision=False):
    return _bwd(y_grad, q, k, v, y, lse, _sca(chunk_size, reset_chunk_pos_per_seq, False), scale, prev_k, prev_v,
                q_segment_idx, k_segment_idx, backend, fp32_kv_grads, high_precision)


@_export
def _flash_sca_sm90_strict_past_fwd(q, k, v, chunk_size, scale, prev_k=None, prev_v=None, q_segment_idx=None,
                                    k_segment_idx=None, backend="auto", reset_chunk_pos_per_seq=False,
                                    output_state=None, high_precision=False):
    return _fwd(q, k, v, _sca(chunk_size, reset_chunk_pos_per_seq, True), scale, prev_k, prev_v, q_segment_idx,
                k_segment_idx, backend, output_state, high_precision)


@_export
def _flash_sca_sm90_strict_past_bwd(y_grad, q, k, v, y, lse, chunk_size, scale, prev_k=None, prev_v=None,
                                    q_segment_idx=None, k_segment_idx=None, deterministic=False, backend="auto",
                                    reset_chunk_pos_per_seq=False, high_precision=False):
    return _bwd(y_grad, q, k, v, y, lse, _sca(chunk_size, reset_chunk_pos_per_seq, True), scale, prev_k, prev_v,
                q_segment_idx, k_segment_idx, backend, high_precision=high_precision)


@_export
def _flash_sca_sm90_varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, chunk_size, scale,
                               position_offsets=None, reset_chunk_pos_per_seq=True, k_run_starts=None,
                               k_run_lengths=None, strict_past=False, output_state=None, high_precision=False):
    """Packed sequences whose chunk positions restart per sequence (the packed layout has no other form
    here: ``position_offsets`` and the K run tables belong to the reference's row-aligned route)."""
    if position_offsets is not None or k_run_starts is not None or k_run_lengths is not None or not reset_chunk_pos_per_seq:
        raise RuntimeError("xattn_cuda: packed sliding-chunk attention restarts positions per sequence; "
                           "row-aligned metadata is not part of this build")
    support = Support("chunk", int(chunk_size), False, bool(strict_past))
    return _varlen.varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, support, float(scale),
                                  output_state=output_state, high_precision=bool(high_precision))


@_export
def _flash_sca_sm90_varlen_bwd(y_grad, q, k, v, y, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                               chunk_size, scale, deterministic=False, position_offsets=None,
                               reset_chunk_pos_per_seq=True, k_run_starts=None, k_run_lengths=None,
                               k_prefix_ends=None, k_row_length=0, strict_past=False):
    if position_offsets is not None or k_run_starts is not None or k_run_lengths is not None or not reset_chunk_pos_per_seq:
        raise RuntimeError("xattn_cuda: packed sliding-chunk attention restarts positions per sequence; "
                           "row-aligned metadata is not part of this build")
    support = Support("chunk", int(chunk_size), False, bool(strict_past))
    return _varlen.varlen_backward(y_grad, q, k, v, y, lse, cu_seqlens_q, cu_seqlens_k, support, float(scale))


@_export
def _flash_sca_sm90_bos_to_segment_idx(bos):
    """int64 segment ids from a BOS mask: a running count of its set bits (xattn/ops/_bos_metadata.py:84-90)."""
    return bos.cumsum(dim=1, dtype=torch.int64)


@_export
def _flash_sca_sm90_bos_to_cu_seqlens(bos):
    """(cu_seqlens int32 over the flattened [B * L] tokens, longest run): every batch row starts a run
    whether or not its first bit is set.  Reads the mask back to the host, as the reference's op does."""
    b, length = bos.shape
    starts = bos.clone()
    starts[:, 0] = True
    flat = starts.reshape(-1).nonzero().flatten().to(torch.int32)
    cu = torch.cat((flat, torch.tensor([b * length], dtype=torch.int32, device=bos.device)))
    return cu, int((cu[1:] - cu[:-1]).max().item())


@_export
def _flash_sca_sm90_clear_inference_bos_fwd_plan_cache():
    """Drops the calling thread's cached mask plans (the plan cache of xattn_b200.ops._core)."""
    _core.clear_plan_cache()


# ---- SoftDelta gate and merge (csrc/softdelta/bindings.cc:11-31) ---------------------------------

@_export
def _softdelta_gate_fwd(read, neg_read, gate, output=None):
    """read - sigmoid(gate) * neg_read, into ``output`` when given."""
    return _native.softdelta_gate_fwd(read, neg_read, gate, out=output)


@_export
def _softdelta_gate_restore(y, neg_read, gate):
    """The query read back from the gated output: y + sigmoid(gate) * neg_read."""
    return _native.softdelta_gate_bwd(torch.zeros_like(y), y, neg_read, gate)[0]


@_export
def _softdelta_gate_bwd(dy, neg_read, gate):
    """(neg_read_grad, gate_grad)."""
    _, dneg, dg = _native.softdelta_gate_bwd(dy, torch.zeros_like(dy), neg_read, gate)
    return dneg, dg


@_export
def _softdelta_merge_gradients(read_key_grad, neg_read_key_grad, dneg_q, read_value_grad, neg_read_value_grad):
    """In place into the read gradients: dK = dK_read + dK_neg (+ the second reader's own gradient on the
    aligned keys, the last rows), dV = dV_read + dV_neg; FP32 sums rounded once."""
    tail = dneg_q if dneg_q is not None and dneg_q.numel() else None
    read_key_grad.copy_(_native.softdelta_merge_gradients(read_key_grad, neg_read_key_grad, tail))
    read_value_grad.copy_(_native.softdelta_merge_gradients(read_value_grad, neg_read_value_grad))
    return read_key_grad, read_value_grad


OP_NAMES = tuple(sorted(name for name in vars(ops) if not name.startswith("__")))
