"""Parity cases shared by the CPU and GPU tests.

The matrix follows the reference's own (tests/_numerics.py:22-81): singleton, uneven head dims,
segment ids, BOS masks, decode, short right-aligned Q (paired / independent / segment / BOS ids),
rows without keys, future-only keys, non-contiguous input layouts, previous K/V, window 0 / 1 /
covering, chunk 1 / unaligned / wide, per-segment reset variants.  Inputs follow
tests/_numerics.py:102-125 (unit-norm q and k, v = silu(randn) + 0.1, dy = randn / sqrt(numel)).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, replace
from typing import Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class Case:
    name: str
    q_length: int = 193
    k_length: int = 193
    dim: int = 64
    value_dim: int = 64
    metadata: str = "dense"      # dense | segment | bos | paired | independent | unmatched | future | long_run
    previous: int = 0
    span: int = 64
    reset: bool = False
    layout: str = "contiguous"   # contiguous | head_slice | offset | last_stride | broadcast
    batch: int = 2
    segment_length: int = 67


BASE_CASES = (
    Case("singleton", 1, 1, 32, 64, batch=1),
    Case("dense-uneven", dim=40, value_dim=56),
    Case("segment", dim=96, value_dim=128, metadata="segment"),
    Case("bos", dim=160, value_dim=192, metadata="bos"),
    Case("decode", 1, 257, 32, 64, batch=1),
    Case("short-paired", 17, 41, 64, 192, metadata="paired"),
    Case("short-independent", 129, 257, 128, 192, metadata="independent"),
    Case("short-segment", 255, 513, 160, 160, metadata="segment"),
    Case("short-bos", 65, 193, 192, 160, metadata="bos"),
    Case("empty-rows", 17, 41, 64, 64, metadata="unmatched"),
    Case("future-only", 4, 9, 32, 64, metadata="future"),
    Case("head-view", layout="head_slice"),
    Case("offset-view", layout="offset"),
    Case("strided-view", layout="last_stride"),
    Case("broadcast-view", layout="broadcast"),
)


def cases_for(operation: str):
    """operation: 'full' | 'window' | 'chunk'."""
    cases = list(BASE_CASES)
    if operation != "full":
        cases += [
            Case("previous", previous=65, dim=128, value_dim=104),
            Case("short-previous", 17, 41, 64, 192, previous=65, metadata="paired"),
            Case("bos-previous", 65, 193, 192, 96, previous=128, metadata="bos"),
        ]
    if operation == "window":
        cases += [Case("window-zero", span=0), Case("window-one", span=1),
                  Case("covering-window", span=512, previous=37)]
    if operation == "chunk":
        cases += [
            Case("chunk-one", span=1, previous=1),
            Case("chunk-unaligned", 513, 513, 192, 96, previous=255, span=255),
            Case("chunk-wide", 517, 517, 256, 160, previous=257, span=257),
            Case("reset", metadata="segment", reset=True),
            Case("short-reset", 17, 41, 64, 192, metadata="independent", reset=True),
            Case("reset-previous", 65, 193, 192, 160, metadata="bos", previous=128, reset=True),
            Case("reset-unmatched", 17, 41, metadata="unmatched", reset=True),
            Case("reset-long-q-run", 17, 41, metadata="long_run", reset=True),
        ]
        # previous K/V of sliding chunks is exactly one chunk long
        cases = [replace(c, span=c.previous) if c.previous else c for c in cases]
    return tuple(cases)


def seed_of(*parts) -> int:
    return int.from_bytes(hashlib.sha256(":".join(map(str, parts)).encode()).digest()[:4], "little")


def make_inputs(operation: str, case: Case, dtype, kv_heads: int, device, heads: int = 4):
    """[q, k, v] (+ [prev_k, prev_v]) as leaf tensors requiring grad."""
    gen = torch.Generator(device="cpu").manual_seed(seed_of(operation, case.name, dtype, kv_heads))

    def rand(*shape):
        return torch.randn(shape, generator=gen, dtype=torch.float32).to(device=device, dtype=dtype)

    B, Lq, D, V = case.batch, case.q_length, case.dim, case.value_dim
    if case.layout == "head_slice":
        q = F.normalize(rand(B, Lq, heads * 2, D), dim=-1)[:, :, 1::2]
    elif case.layout == "offset":
        q = F.normalize(rand(B, Lq, heads, D + 1), dim=-1)[..., 1:]
    elif case.layout == "last_stride":
        q = F.normalize(rand(B, Lq, heads, D * 2), dim=-1)[..., ::2]
    elif case.layout == "broadcast":
        q = F.normalize(rand(B, Lq, 1, D), dim=-1).expand(B, Lq, heads, D)
    else:
        q = F.normalize(rand(B, Lq, heads, D), dim=-1)
    total = case.k_length + case.previous
    kt = F.normalize(rand(B, total, kv_heads, D), dim=-1)
    vt = F.silu(rand(B, total, kv_heads, V)) + 0.1
    tensors = [q, kt[:, case.previous:], vt[:, case.previous:]]
    if case.previous:
        tensors += [kt[:, :case.previous], vt[:, :case.previous]]
    return [t.detach().requires_grad_() for t in tensors]


def metadata_for(case: Case, device):
    """(options for the public op, q ids, k ids) — ids are None for dense cases."""
    options = {}
    qi = ki = None
    if case.metadata == "dense":
        return options, qi, ki
    total = case.k_length + case.previous
    ki = (torch.arange(total, device=device) // case.segment_length).expand(case.batch, -1).clone()
    ki += torch.arange(case.batch, device=device)[:, None] * 100
    qi = ki[:, -case.q_length:].clone()
    if case.metadata == "independent":
        qi[:, :min(max(1, case.q_length // 3), 33)] = ki[:, :1]
    elif case.metadata == "unmatched":
        qi.fill_(-1)
    elif case.metadata == "long_run":
        qi = ki[:, :1].expand(case.batch, case.q_length).clone()
    elif case.metadata == "future":
        ki.zero_()
        ki[:, -3:] = 1
        qi.fill_(1)
    if case.metadata == "segment":
        options["segment_idx"] = ki
    elif case.metadata == "bos":
        bos = torch.ones_like(ki, dtype=torch.bool)
        bos[:, 1:] = ki[:, 1:] != ki[:, :-1]
        options["bos_mask"] = bos
    else:
        options.update(q_segment_idx=qi, k_segment_idx=ki)
    return options, qi, ki


def op_options(operation: str, case: Case, inputs):
    options = {}
    if operation == "window":
        options["window_size"] = case.span
    elif operation == "chunk":
        options.update(chunk_size=case.span, reset_chunk_pos_per_seq=case.reset)
    if case.previous:
        options.update(prev_k=inputs[-2], prev_v=inputs[-1])
    return options
