"""Generates tests/golden/attention_golden.npz from the REFERENCE's own oracle.

Run once where a checkout of the reference is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's tests/_reference.py (``_allowed_masks``, ``_attention_from_mask``) and
tests/softdelta/reference.py (``softdelta_fp64_oracle``), runs them in FP64 on small seeded inputs
(numpy RandomState, so the inputs can be rebuilt anywhere) and stores masks, outputs and gradients.
tests/test_oracle.py checks oracle/attention_oracle.py against the stored values; nothing at test
time needs the reference checkout.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from golden_cases import GOLDEN_CASES, golden_inputs  # noqa: E402


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    from tests._reference import _allowed_masks, _attention_from_mask  # reference code
    from tests.softdelta.reference import softdelta_fp64_oracle        # reference code

    out = {}
    for case in GOLDEN_CASES:
        t = golden_inputs(case)
        q, k, v, dy = (t[n].clone().requires_grad_(n != "dy") for n in ("q", "k", "v", "dy"))
        inc, strict = _allowed_masks(case["Lq"], case["Lk"], case["B"], torch.device("cpu"), case["vis"],
                                     case["span"], t["q_ids"], t["k_ids"], case["reset"])
        mask = strict if case["strict"] else inc
        scale = case["D"] ** -0.5
        y = _attention_from_mask(q, k, v, mask, scale)
        dq, dk, dv = torch.autograd.grad(y, (q, k, v), dy)
        name = case["name"]
        out[name + "/inclusive"] = np.packbits(inc.numpy())
        out[name + "/strict"] = np.packbits(strict.numpy())
        for key, val in (("y", y), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[f"{name}/{key}"] = val.detach().numpy().astype(np.float64)
        if case.get("softdelta"):
            g = t["g"].clone().requires_grad_()
            q2, k2, v2 = (t[n].clone().requires_grad_() for n in ("q", "k", "v"))
            dy2 = dy
            if case.get("groups"):       # the reference's internal value-group layout
                shape = (case["groups"], case["V"] // case["groups"])
                v2 = t["v"].unflatten(3, shape).clone().requires_grad_()
                dy2 = dy.unflatten(3, shape)
            ys = softdelta_fp64_oracle(q2, k2, v2, g, None, scale=scale, q_segment_idx=t["q_ids"],
                                       k_segment_idx=t["k_ids"], visibility=case["vis"], span=case["span"],
                                       reset_position_per_segment=case["reset"])
            grads = torch.autograd.grad(ys, (q2, k2, v2, g), dy2)
            out[name + "/sd_y"] = ys.detach().numpy()
            for key, val in zip(("sd_dq", "sd_dk", "sd_dv", "sd_dg"), grads):
                out[f"{name}/{key}"] = val.numpy()
    path = os.path.join(HERE, "attention_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
