"""Small seeded cases behind tests/golden/attention_golden.npz (shared by the generator and the test)."""
from __future__ import annotations

import zlib

import numpy as np
import torch


def _case(name, B, Lq, Lk, Hq, Hkv, D, V, vis="full", span=None, seg=None, reset=False, strict=False,
          q_ids="suffix", softdelta=False, groups=None):
    """``groups``: SoftDelta value groups (v seen as [.., groups, V / groups], one gate per group)."""
    return dict(name=name, B=B, Lq=Lq, Lk=Lk, Hq=Hq, Hkv=Hkv, D=D, V=V, vis=vis, span=span, seg=seg,
                reset=reset, strict=strict, q_ids=q_ids, softdelta=softdelta, groups=groups)


GOLDEN_CASES = (
    _case("causal", 2, 24, 24, 2, 2, 8, 8, softdelta=True),
    _case("causal-gqa", 1, 20, 20, 4, 2, 8, 16),
    _case("causal-mqa-short-q", 2, 7, 19, 4, 1, 8, 8),
    _case("causal-strict", 1, 16, 16, 2, 1, 8, 8, strict=True),
    _case("window-3", 2, 20, 20, 2, 1, 8, 8, vis="window", span=3, softdelta=True),
    _case("window-0", 1, 12, 12, 2, 2, 8, 8, vis="window", span=0),
    _case("window-short-q", 1, 5, 17, 2, 1, 8, 8, vis="window", span=4),
    _case("chunk-4", 2, 21, 21, 2, 2, 8, 8, vis="chunk", span=4, softdelta=True),
    _case("chunk-1", 1, 9, 9, 2, 1, 8, 8, vis="chunk", span=1),
    _case("chunk-short-q", 1, 6, 18, 2, 2, 8, 8, vis="chunk", span=5),
    _case("segment", 2, 22, 22, 2, 1, 8, 8, seg=7, softdelta=True),
    _case("segment-short-q", 2, 9, 22, 2, 2, 8, 8, seg=7),
    _case("segment-window", 1, 22, 22, 2, 2, 8, 8, vis="window", span=3, seg=6),
    _case("segment-chunk-reset", 2, 23, 23, 2, 1, 8, 8, vis="chunk", span=3, seg=8, reset=True, softdelta=True),
    _case("segment-chunk-global", 1, 23, 23, 2, 1, 8, 8, vis="chunk", span=3, seg=8),
    _case("reset-independent", 2, 9, 23, 2, 1, 8, 8, vis="chunk", span=3, seg=8, reset=True, q_ids="independent"),
    _case("reset-long-q-run", 1, 9, 23, 2, 1, 8, 8, vis="chunk", span=3, seg=8, reset=True, q_ids="long_run"),
    _case("unmatched", 1, 6, 14, 2, 1, 8, 8, seg=5, q_ids="unmatched"),
    _case("future-only", 1, 4, 9, 2, 1, 8, 8, seg=5, q_ids="future"),
    _case("groups-causal", 2, 18, 18, 4, 2, 8, 12, softdelta=True, groups=3),
    _case("groups-segment-window", 1, 20, 20, 2, 1, 8, 16, vis="window", span=4, seg=6, softdelta=True, groups=2),
)


def golden_inputs(case):
    """FP64 torch tensors q, k, v, dy, g and int64 ids (or None), rebuilt from the case name."""
    rs = np.random.RandomState(zlib.crc32(case["name"].encode()) & 0x7FFFFFFF)
    B, Lq, Lk, Hq, Hkv, D, V = (case[n] for n in ("B", "Lq", "Lk", "Hq", "Hkv", "D", "V"))
    t = {
        "q": torch.from_numpy(rs.standard_normal((B, Lq, Hq, D))),
        "k": torch.from_numpy(rs.standard_normal((B, Lk, Hkv, D))),
        "v": torch.from_numpy(rs.standard_normal((B, Lk, Hkv, V))),
        "dy": torch.from_numpy(rs.standard_normal((B, Lq, Hq, V))),
        "g": torch.from_numpy(rs.standard_normal((B, Lq, Hq) if not case.get("groups") else
                                                 (B, Lq, Hq, case["groups"], 1))),
        "q_ids": None,
        "k_ids": None,
    }
    if case["seg"]:
        ki = (torch.arange(Lk) // case["seg"]).expand(B, -1).clone() + torch.arange(B)[:, None] * 100
        qi = ki[:, -Lq:].clone()
        mode = case["q_ids"]
        if mode == "independent":
            qi[:, :max(1, Lq // 3)] = ki[:, :1]
        elif mode == "long_run":
            qi = ki[:, :1].expand(B, Lq).clone()
        elif mode == "unmatched":
            qi.fill_(-1)
        elif mode == "future":
            ki.zero_()
            ki[:, -3:] = 1
            qi.fill_(1)
        t["q_ids"], t["k_ids"] = qi, ki
    return t
