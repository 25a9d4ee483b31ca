"""torch-facing wrappers of the C ABI: allocate outputs and workspaces, pass raw
pointers, turn status codes into exceptions.

This is the part of the reference's pybind layer that stays in Python
(csrc/causal_flash_attn/causal_flash_attn.cc:49-122 and friends allocate the
outputs and forward the tensors; here the library only ever sees pointers).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib

_DTYPES = {torch.float16: _lib.XATTN_DTYPE_F16, torch.bfloat16: _lib.XATTN_DTYPE_BF16}
_VIS = {"full": _lib.VIS_FULL, "window": _lib.VIS_WINDOW, "chunk": _lib.VIS_CHUNK, "all": _lib.VIS_ALL}

# XATTN_B200_SYNC_CHECK=1: read the device status word after every launch
# (synchronises).  Otherwise the word is read back asynchronously and examined
# at the next call on the same device.
_SYNC_CHECK = os.environ.get("XATTN_B200_SYNC_CHECK", "0") == "1"


class _DeviceState:
    def __init__(self, device: torch.device):
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None


_states = {}


def _state(device: torch.device) -> _DeviceState:
    index = device.index if device.index is not None else torch.cuda.current_device()
    st = _states.get(index)
    if st is None:
        st = _states[index] = _DeviceState(torch.device("cuda", index))
    return st


def prepare_device(device: Optional[torch.device] = None) -> None:
    """Create this module's per-device state now: the device status word (4 bytes) and its pinned host
    mirror.  Every entry point does this on first use; callers of ``attention_bwd_static_scratch``, which
    may not allocate later on, call it once at start-up instead."""
    _state(torch.device("cuda", torch.cuda.current_device()) if device is None else device)


def _stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _raise_status(value: int) -> None:
    if value & 0xff == 3:
        raise RuntimeError(
            f"segment ids of the keys decrease along batch row {value >> 8}: k_segment_idx / segment_idx must "
            "be nondecreasing along each row (the keys of one id are located by binary search); results "
            "of that call are invalid"
        )
    raise RuntimeError(
        f"xattn_b200 kernel reported device status {value & 0xff} at wait site {value >> 8}; "
        "results of that launch are invalid"
    )


def _pre_launch(device: torch.device) -> _DeviceState:
    st = _state(device)
    if torch.cuda.is_current_stream_capturing():
        return st    # no event queries inside a CUDA graph capture; check_status() after a replay reads the word
    if st.event is not None and st.event.query():
        st.event = None
        value = int(st.host[0])
        if value:
            st.status.zero_()
            _raise_status(value)
    return st


def _post_launch(st: _DeviceState) -> None:
    if torch.cuda.is_current_stream_capturing():
        return
    if _SYNC_CHECK:
        torch.cuda.current_stream().synchronize()
        value = int(st.status.item())
        if value:
            st.status.zero_()
            _raise_status(value)
        return
    if st.event is None:
        st.host.copy_(st.status, non_blocking=True)
        st.event = torch.cuda.Event()
        st.event.record()


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel launched so far reported a device-side status."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    st = _state(device)
    torch.cuda.synchronize(device)
    st.event = None
    value = int(st.status.item())
    if value:
        st.status.zero_()
        _raise_status(value)


def selftest_wait_timeout(device: torch.device, budget_us: int = 2000) -> None:
    """Launch the library's wait-timeout probe on ``device``: a kernel whose wait runs out after
    ``budget_us`` microseconds and reports it in the device status word, exactly as a stuck tensor
    kernel would.  The next status check on that device (``check_status()``, or the next launch)
    raises."""
    lib = _lib.load()
    with torch.cuda.device(device):
        st = _pre_launch(device)
        _lib.check(lib.xattn_b200_selftest_wait_timeout(st.status.data_ptr(), int(budget_us), _stream_ptr()),
                   "xattn_b200_selftest_wait_timeout")
        _post_launch(st)


def require_cuda(t: Tensor, api_name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{api_name} needs CUDA tensors; this build has no CPU path")
    major, _ = torch.cuda.get_device_capability(t.device)
    if major != 10:
        raise RuntimeError(f"{api_name} is built for sm_100a only (device capability {major}.x found)")


def tma_ready(t: Tensor) -> Tensor:
    """Return ``t`` itself when TMA can read it in place (unit last stride, 16-byte aligned base and
    strides — the rule of csrc/causal_attention/launch.cu:85-95), otherwise a contiguous copy."""
    if t.dim() >= 1 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0:
        ok = True
        for size, stride in zip(t.shape[:-1], t.stride()[:-1]):
            if size > 1 and (stride <= 0 or (stride * t.element_size()) % 16):
                ok = False
                break
        if ok:
            return t
    out = t.contiguous()
    if out.data_ptr() % 16:
        out = out.clone(memory_format=torch.contiguous_format)
    return out


def plan_bytes(batch: int, q_len: int, k_len: int) -> int:
    return int(_lib.load().xattn_b200_plan_bytes(batch, q_len, k_len))


def build_plan(
    batch: int,
    q_len: int,
    k_len: int,
    device: torch.device,
    *,
    visibility: str = "full",
    span: Optional[int] = None,
    strict_past: bool = False,
    reset_positions: bool = False,
    q_segment_idx: Optional[Tensor] = None,
    k_segment_idx: Optional[Tensor] = None,
) -> Tensor:
    """Device plan (int32 tensor) for dense [B, L, H, D] inputs."""
    lib = _lib.load()
    plan = torch.empty(plan_bytes(batch, q_len, k_len) // 4, dtype=torch.int32, device=device)
    args = _lib.PlanArgs()
    args.batch, args.q_len, args.k_len = batch, q_len, k_len
    args.visibility = _VIS[visibility]
    args.span = 0 if span is None else int(span)
    args.strict_past = int(bool(strict_past))
    args.reset_positions = int(bool(reset_positions))
    keep = []
    if q_segment_idx is not None:
        qs = q_segment_idx if q_segment_idx.stride(-1) == 1 else q_segment_idx.contiguous()
        ks = k_segment_idx if k_segment_idx.stride(-1) == 1 else k_segment_idx.contiguous()
        keep += [qs, ks]
        args.q_segment, args.k_segment = qs.data_ptr(), ks.data_ptr()
        args.q_segment_stride = qs.stride(0) if batch > 1 else q_len
        args.k_segment_stride = ks.stride(0) if batch > 1 else k_len
    args.plan = plan.data_ptr()
    with torch.cuda.device(device):
        st = None
        # The sorted-ids check reads every key id once more: skipped for decode shapes, where that pass
        # would cost more than the plan itself.
        if q_segment_idx is not None and not (q_len <= 128 and k_len > 4096):
            st = _pre_launch(device)
            args.status = st.status.data_ptr()
        _lib.check(lib.xattn_b200_build_plan(C.byref(args), _stream_ptr()), "xattn_b200_build_plan")
        if st is not None:
            _post_launch(st)
    return plan


def build_varlen_plan(
    cu_seqlens_q: Tensor,
    cu_seqlens_k: Tensor,
    total_q: int,
    total_k: int,
    *,
    visibility: str = "full",
    span: Optional[int] = None,
    strict_past: bool = False,
) -> Tensor:
    lib = _lib.load()
    device = cu_seqlens_q.device
    plan = torch.empty(plan_bytes(1, total_q, total_k) // 4, dtype=torch.int32, device=device)
    args = _lib.VarlenPlanArgs()
    args.total_q, args.total_k = total_q, total_k
    args.num_q_seqs, args.num_k_seqs = cu_seqlens_q.numel() - 1, cu_seqlens_k.numel() - 1
    cq, ck = cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous()
    args.cu_seqlens_q, args.cu_seqlens_k = cq.data_ptr(), ck.data_ptr()
    args.visibility = _VIS[visibility]
    args.span = 0 if span is None else int(span)
    args.strict_past = int(bool(strict_past))
    args.plan = plan.data_ptr()
    with torch.cuda.device(device):
        _lib.check(lib.xattn_b200_build_varlen_plan(C.byref(args), _stream_ptr()), "xattn_b200_build_varlen_plan")
    return plan


def attention_fwd(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    plan: Tensor,
    scale: float,
    *,
    high_precision: bool = False,
    output_state: Optional[Tensor] = None,
    splits: Optional[int] = None,
    return_anchor: bool = False,
):
    """y [B,Lq,Hq,V] (input dtype), lse [B,Hq,Lq] fp32.  ``k``/``v`` already include previous K/V.
    With ``return_anchor`` (high precision only) a third result: int32 [B,Hq,Lq], the visible key
    holding each row's largest logit, which the high-precision backward centres dP on.

    Decode shapes (a few query rows against many keys) take the split entry, which shares a tile among
    the query heads of a KV group and divides the keys among CTAs; ``splits`` overrides the library's
    choice (0: never split).
    """
    lib = _lib.load()
    require_cuda(q, "xattn_b200 forward")
    q, k, v = tma_ready(q), tma_ready(k), tma_ready(v)
    B, Lq, Hq, D = q.shape
    Lk, Hkv, V = k.shape[1], k.shape[2], v.shape[3]
    y = torch.empty((B, Lq, Hq, V), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Lq), dtype=torch.float32, device=q.device)
    args = _lib.FwdArgs()
    args.dtype = _DTYPES[q.dtype]
    args.batch, args.q_len, args.k_len = B, Lq, Lk
    args.q_heads, args.kv_heads, args.qk_dim, args.v_dim = Hq, Hkv, D, V
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v)):
        setattr(args, name, (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2)))
    args.scale = float(scale)
    args.high_precision = int(bool(high_precision))
    args.plan = plan.data_ptr()
    args.y, args.lse = y.data_ptr(), lse.data_ptr()
    if output_state is not None:
        if output_state.shape != y.shape or output_state.dtype != torch.float32 or not output_state.is_contiguous():
            raise ValueError("output_state must be a contiguous FP32 tensor shaped like y")
        args.y_state = output_state.data_ptr()
    anchor = None
    if return_anchor:
        if not high_precision:
            raise ValueError("anchor keys are a result of the high-precision forward only")
        anchor = torch.empty((B, Hq, Lq), dtype=torch.int32, device=q.device)
        args.anchor = anchor.data_ptr()
        splits = 0          # the split forward of decode shapes does not track anchors
    with torch.cuda.device(q.device):
        st = _pre_launch(q.device)
        args.status = st.status.data_ptr()
        if splits is None:
            splits = int(lib.xattn_b200_fwd_split_suggest(B, Lq, Lk, Hq, Hkv, st.sm_count))
        if splits > 0:
            nbytes = int(lib.xattn_b200_fwd_split_workspace_bytes(B, Lq, Hq, V, splits))
            workspace = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
            _lib.check(lib.xattn_b200_fwd_split(C.byref(args), splits, workspace.data_ptr(), nbytes, _stream_ptr()),
                       "xattn_b200_fwd_split")
        else:
            _lib.check(lib.xattn_b200_fwd(C.byref(args), _stream_ptr()), "xattn_b200_fwd")
        _post_launch(st)
    return (y, lse, anchor) if return_anchor else (y, lse)


class BackwardCall:
    """One backward of ``attention_fwd``'s result, runnable in phases.

    ``run()`` launches the whole backward.  ``run(_lib.BWD_PHASE_PRE | _lib.BWD_PHASE_DKV)`` followed by
    ``run(_lib.BWD_PHASE_DQ)`` launches dK / dV first, so that a caller can start sending parts of them
    (the K/V halo's gradients of a sequence-sharded run) while the dQ kernel runs.  Outputs ``dq``,
    ``dk``, ``dv`` (shaped like q, k, v with previous K/V included, input dtype) and the workspace are
    allocated here once and shared by the phases."""

    def __init__(self, dy: Tensor, q: Tensor, k: Tensor, v: Tensor, y: Tensor, lse: Tensor, plan: Tensor,
                 scale: float, *, anchor: Optional[Tensor] = None, grad_unscale: Optional[Tensor] = None):
        lib = _lib.load()
        require_cuda(q, "xattn_b200 backward")
        q, k, v, y, dy = tma_ready(q), tma_ready(k), tma_ready(v), tma_ready(y), tma_ready(dy)
        lse = lse.contiguous()
        B, Lq, Hq, D = q.shape
        Lk, Hkv, V = k.shape[1], k.shape[2], v.shape[3]
        self.dq = torch.empty((B, Lq, Hq, D), dtype=q.dtype, device=q.device)
        self.dk = torch.empty((B, Lk, Hkv, D), dtype=q.dtype, device=q.device)
        self.dv = torch.empty((B, Lk, Hkv, V), dtype=q.dtype, device=q.device)
        nbytes = lib.xattn_b200_bwd_workspace_bytes_hp if anchor is not None else lib.xattn_b200_bwd_workspace_bytes
        ws = torch.empty(int(nbytes(B, Hq, Lq)) // 4, dtype=torch.float32, device=q.device)
        args = _lib.BwdArgs()
        args.dtype = _DTYPES[q.dtype]
        args.batch, args.q_len, args.k_len = B, Lq, Lk
        args.q_heads, args.kv_heads, args.qk_dim, args.v_dim = Hq, Hkv, D, V
        args.q, args.k, args.v, args.y, args.dy = q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), dy.data_ptr()
        for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("y_strides", y), ("dy_strides", dy)):
            setattr(args, name, (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2)))
        args.lse = lse.data_ptr()
        args.scale = float(scale)
        args.plan = plan.data_ptr()
        args.dq, args.dk, args.dv = self.dq.data_ptr(), self.dk.data_ptr(), self.dv.data_ptr()
        args.workspace = ws.data_ptr()
        if anchor is not None:
            if anchor.shape != (B, Hq, Lq) or anchor.dtype != torch.int32 or not anchor.is_contiguous():
                raise ValueError("anchor must be a contiguous int32 tensor [B, Hq, Lq]")
            args.high_precision = 1
            args.anchor = anchor.data_ptr()
        if grad_unscale is not None:
            if grad_unscale.dtype != torch.float32 or grad_unscale.numel() != 1 or grad_unscale.device != q.device:
                raise ValueError("grad_unscale must be one FP32 number on the inputs' device")
            args.grad_unscale = grad_unscale.data_ptr()
        self._args, self._device = args, q.device
        self._keep = (q, k, v, y, dy, lse, plan, ws, anchor, grad_unscale)    # alive until the last phase has run

    def run(self, phases: int = 0) -> "BackwardCall":
        lib = _lib.load()
        self._args.phases = int(phases)
        with torch.cuda.device(self._device):
            st = _pre_launch(self._device)
            self._args.status = st.status.data_ptr()
            _lib.check(lib.xattn_b200_bwd(C.byref(self._args), _stream_ptr()), "xattn_b200_bwd")
            _post_launch(st)
        return self


def attention_bwd(
    dy: Tensor,
    q: Tensor,
    k: Tensor,
    v: Tensor,
    y: Tensor,
    lse: Tensor,
    plan: Tensor,
    scale: float,
    *,
    anchor: Optional[Tensor] = None,
    grad_unscale: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor, Tensor]:
    """(dq, dk, dv) shaped like q, k, v (k / v including previous K/V), in the input dtype.

    With ``anchor`` (and ``lse``) from the high-precision forward on the same inputs this is the
    high-precision backward: dP centred on each row's anchor key, the row statistic recomputed from
    centred terms, P formed as a square of its root (xattn/ops/_precision_backend.py:29-170).
    ``grad_unscale``: optional FP32 device scalar multiplied into the three gradients before they are
    rounded (undoes a power-of-two prescale of ``dy``)."""
    call = BackwardCall(dy, q, k, v, y, lse, plan, scale, anchor=anchor, grad_unscale=grad_unscale).run()
    return call.dq, call.dk, call.dv


def zero_constant_key_rows(dq: Tensor, k_all: Tensor, plan: Tensor) -> Tensor:
    """Level-1 repair, in place on ``dq`` (contiguous): rows whose visible keys are one repeated
    vector get an exactly zero gradient."""
    lib = _lib.load()
    k_all = tma_ready(k_all)
    B, Lq, Hq, D = dq.shape
    Lk, Hkv = k_all.shape[1], k_all.shape[2]
    ws = torch.empty(B * Hkv * Lk, dtype=torch.int32, device=dq.device)
    args = _lib.ConstantKeyArgs()
    args.dtype = _DTYPES[dq.dtype]
    args.batch, args.q_len, args.k_len, args.q_heads, args.kv_heads, args.qk_dim = B, Lq, Lk, Hq, Hkv, D
    args.dq, args.k = dq.data_ptr(), k_all.data_ptr()
    args.k_strides = (C.c_int64 * 3)(k_all.stride(0), k_all.stride(1), k_all.stride(2))
    args.plan, args.workspace = plan.data_ptr(), ws.data_ptr()
    with torch.cuda.device(dq.device):
        _lib.check(lib.xattn_b200_zero_constant_key_rows(C.byref(args), _stream_ptr()),
                   "xattn_b200_zero_constant_key_rows")
    return dq


def softdelta_merge_gradients(a: Tensor, b: Tensor, tail: Optional[Tensor] = None) -> Tensor:
    """a + b (+ ``tail`` on the last rows of every batch row), summed in FP32 and rounded once; [B, L, H, D]
    tensors of the input dtype.  Returns a new tensor."""
    lib = _lib.load()
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty_like(a)
    args = _lib.MergeArgs()
    args.dtype = _DTYPES[a.dtype]
    args.batch, args.k_len, args.kv_heads, args.dim = a.shape
    args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    if tail is not None:
        tail = tail.contiguous()
        args.tail, args.tail_len = tail.data_ptr(), tail.shape[1]
    with torch.cuda.device(a.device):
        _lib.check(lib.xattn_b200_softdelta_merge_gradients(C.byref(args), _stream_ptr()),
                   "xattn_b200_softdelta_merge_gradients")
    return out


def _gate_args(g: Tensor, neg_read: Tensor, q_heads: int) -> "_lib.GateArgs":
    """``g`` is [B, L, H] (one gate per head) or [B, L, H, C] (one per group of V / C channels)."""
    args = _lib.GateArgs()
    args.dtype = _DTYPES[g.dtype]
    args.neg_is_f32 = int(neg_read.dtype == torch.float32)
    B, L, Hkv, V = neg_read.shape
    args.rows, args.q_heads, args.kv_heads, args.v_dim = B * L, q_heads, Hkv, V
    args.value_groups = g.shape[3] if g.dim() == 4 else 1
    args.g, args.neg_read = g.data_ptr(), neg_read.data_ptr()
    return args


def softdelta_gate_fwd(read: Tensor, neg_read: Tensor, g: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """y = read - sigmoid(g) * neg_read; ``out`` may be ``read`` itself."""
    lib = _lib.load()
    read, neg_read, g = read.contiguous(), neg_read.contiguous(), g.contiguous()
    y = torch.empty_like(read) if out is None else out
    args = _gate_args(g, neg_read, read.shape[2])
    args.read, args.y = read.data_ptr(), y.data_ptr()
    with torch.cuda.device(read.device):
        _lib.check(lib.xattn_b200_softdelta_gate_fwd(C.byref(args), _stream_ptr()), "xattn_b200_softdelta_gate_fwd")
    return y


def softdelta_gate_bwd(dy: Tensor, y: Tensor, neg_read: Tensor, g: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """(read, dneg_read, dg): the recovered query read and the gate's gradients, one pass."""
    lib = _lib.load()
    dy, y, neg_read, g = dy.contiguous(), y.contiguous(), neg_read.contiguous(), g.contiguous()
    read = torch.empty_like(y)
    dneg = torch.empty(neg_read.shape, dtype=y.dtype, device=y.device)
    dg = torch.empty_like(g)
    args = _gate_args(g, neg_read, y.shape[2])
    args.read, args.y, args.dy = read.data_ptr(), y.data_ptr(), dy.data_ptr()
    args.dneg_read, args.dg = dneg.data_ptr(), dg.data_ptr()
    with torch.cuda.device(y.device):
        _lib.check(lib.xattn_b200_softdelta_gate_bwd(C.byref(args), _stream_ptr()), "xattn_b200_softdelta_gate_bwd")
    return read, dneg, dg


def merge_partial_outputs(y_acc: Tensor, lse_acc: Tensor, y_part: Tensor, lse_part: Tensor, row_offset: int = 0) -> None:
    """Fold a K/V block's normalised FP32 partial output (``y_part`` [B, R, H, V], ``lse_part`` [B, H, R])
    into the running result, in place; the partial result covers the rows from ``row_offset`` on."""
    lib = _lib.load()
    for t in (y_acc, lse_acc, y_part, lse_part):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError("partial outputs and their lse must be contiguous FP32 tensors")
    args = _lib.MergeOutputsArgs()
    args.batch, args.rows, args.heads, args.v_dim = y_part.shape
    args.acc_rows, args.row_offset = y_acc.shape[1], int(row_offset)
    args.y_acc, args.lse_acc = y_acc.data_ptr(), lse_acc.data_ptr()
    args.y_part, args.lse_part = y_part.data_ptr(), lse_part.data_ptr()
    with torch.cuda.device(y_acc.device):
        _lib.check(lib.xattn_b200_merge_partial_outputs(C.byref(args), _stream_ptr()), "xattn_b200_merge_partial_outputs")


PROFILE_KINDS = {1: "plan", 2: "fwd", 3: "bwd_pre", 4: "bwd_dq", 5: "bwd_dkv", 6: "gate", 7: "repair",
                 8: "bwd_stats"}


def profile_enable(enable: bool) -> None:
    """Bracket every kernel launched by the library with CUDA events (for benchmarks)."""
    _lib.load().xattn_b200_profile_enable(int(bool(enable)))


def profile_read(capacity: int = 65536):
    """[(kind name, milliseconds)] of the launches since the last read; synchronises their events."""
    kinds = (C.c_int * capacity)()
    ms = (C.c_float * capacity)()
    n = _lib.load().xattn_b200_profile_read(kinds, ms, capacity)
    return [(PROFILE_KINDS.get(kinds[i], str(kinds[i])), float(ms[i])) for i in range(max(n, 0))]


STATIC_SCRATCH_MAX_ROWS = 1 << 20


def attention_bwd_static_scratch(dy: Tensor, q: Tensor, k: Tensor, v: Tensor, y: Tensor, lse: Tensor,
                                 plan: Tensor, scale: float, dq: Tensor, dk: Tensor, dv: Tensor) -> None:
    """Backward into caller-provided ``dq`` / ``dk`` / ``dv`` without any device allocation.

    For callers that are not allowed to allocate on the device (a host application that owns all
    device memory and passes an op only its inputs and outputs; a serving loop that must not hit
    the device-wide stall of an allocation).  The kernel scratch is a fixed array inside the
    library instead of a tensor, so ``batch * q_heads * q_len`` (``q_len`` rounded up to a
    multiple of 128) is limited to ``STATIC_SCRATCH_MAX_ROWS``; calls on one device share that array and must not overlap on the
    GPU.  Every tensor must already be laid out the way the kernels read it (unit last stride,
    16-byte aligned base and strides): nothing is copied or made contiguous here.  The first call
    on a device resolves the array's address (and, where CUDA loads modules lazily, loads the module
    and reserves the array): make it at start-up, outside any stream capture.  The device status word
    must exist already: ``prepare_device()`` at start-up, or any earlier call of this module on the
    device, creates it; this function refuses to allocate it.
    """
    lib = _lib.load()
    require_cuda(q, "xattn_b200 backward (static scratch)")
    for name, t in (("q", q), ("k", k), ("v", v), ("y", y), ("dy", dy)):
        if tma_ready(t) is not t:
            raise ValueError(f"{name} needs a unit last stride and 16-byte aligned base and strides; "
                             "this entry point does not copy")
    for name, t in (("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    B, Lq, Hq, D = q.shape
    Lk, Hkv, V = k.shape[1], k.shape[2], v.shape[3]
    if dq.shape != q.shape or dk.shape != k.shape or dv.shape != v.shape:
        raise ValueError("dq / dk / dv must be shaped like q / k / v")
    args = _lib.BwdArgs()
    args.dtype = _DTYPES[q.dtype]
    args.batch, args.q_len, args.k_len = B, Lq, Lk
    args.q_heads, args.kv_heads, args.qk_dim, args.v_dim = Hq, Hkv, D, V
    args.q, args.k, args.v, args.y, args.dy = q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), dy.data_ptr()
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("y_strides", y), ("dy_strides", dy)):
        setattr(args, name, (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2)))
    args.lse = lse.data_ptr()
    args.scale = float(scale)
    args.plan = plan.data_ptr()
    args.dq, args.dk, args.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    args.workspace = None
    index = q.device.index if q.device.index is not None else torch.cuda.current_device()
    if index not in _states:
        raise RuntimeError("the device status word does not exist yet and this entry point may not allocate it: "
                           "call xattn_b200._native.prepare_device() once at start-up")
    with torch.cuda.device(q.device):
        st = _pre_launch(q.device)
        args.status = st.status.data_ptr()
        _lib.check(lib.xattn_b200_bwd_static_scratch(C.byref(args), _stream_ptr()),
                   "xattn_b200_bwd_static_scratch")
        _post_launch(st)
