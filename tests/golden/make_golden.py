"""Generate golden vectors from the REFERENCE implementation itself.

Run once inside a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/flash-window-attention-v2

It imports the reference's classic path (`win_attention_torch`,
flash_win_attn_v2/win_attention_func.py:11-39), runs it in float64 with
autograd on the seeded inputs of `flash_window_attention_v2_b200.workloads`,
and writes one small .npz per case next to this file.  The committed .npz
files are what `tests/test_oracle.py` pins the CPU oracle against; the
reference is not needed to run the tests.
"""
from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from flash_window_attention_v2_b200.workloads import CONFIGS, Workload, make_inputs  # noqa: E402

# name -> (workload, make_inputs kwargs, post-processing tag)
CASES = {
    "cfg1": (CONFIGS["cfg1"], {}, None),
    "n144_ragged": (Workload("n144", batch=1, nw=4, heads=2, window=12, dtype="fp32"), {}, None),
    "n256": (Workload("n256", batch=1, nw=4, heads=2, window=16, dtype="fp32"), {}, None),
    "n64_nomask": (Workload("n64a", batch=1, nw=4, heads=2, window=8, dtype="fp32"), {"with_mask": False}, None),
    "n64_nobias": (Workload("n64b", batch=1, nw=4, heads=2, window=8, dtype="fp32"), {"with_bias": False}, None),
    "n64_scalar": (Workload("n64c", batch=1, nw=4, heads=2, window=8, dtype="fp32"), {"with_scale": False}, None),
    "n64_qkv_only": (Workload("n64d", batch=1, nw=4, heads=2, window=8, dtype="fp32"),
                     {"with_scale": False, "with_bias": False, "with_mask": False}, None),
    "n64_clamped": (Workload("n64e", batch=1, nw=4, heads=2, window=8, dtype="fp32"), {}, "clamp_head0"),
    "n64_infmask": (Workload("n64f", batch=1, nw=4, heads=2, window=8, dtype="fp32"), {}, "inf_mask"),
    "n49": (Workload("n49", batch=1, nw=4, heads=2, window=7, dtype="fp32", shift=3), {}, None),
}


def build_inputs(name: str):
    w, kw, tag = CASES[name]
    t = make_inputs(w, seed=0, **kw)
    if tag == "clamp_head0":
        g = t["logit_scale"].clone()
        g[0] = 5.0  # above ln(100): scale clamps to 100, gradient gated to zero
        t["logit_scale"] = g
    if tag == "inf_mask":
        gen = torch.Generator().manual_seed(1)
        m = torch.zeros_like(t["mask"])
        drop = torch.rand(m.shape, generator=gen) < 0.4
        # keep the diagonal so no row is fully masked
        eye = torch.eye(m.shape[-1], dtype=torch.bool)[None]
        m[drop & ~eye] = float("-inf")
        t["mask"] = m
    return w, t


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    from flash_win_attn_v2.win_attention_func import win_attention_torch  # the reference oracle

    for name in CASES:
        w, t = build_inputs(name)
        q, k, v = (t[x].double().requires_grad_(True) for x in ("q", "k", "v"))
        g = t["logit_scale"].double().requires_grad_(True) if t["logit_scale"] is not None else None
        b = t["bias"].double().requires_grad_(True) if t["bias"] is not None else None
        m = t["mask"].double() if t["mask"] is not None else None
        o = win_attention_torch(q, k, v, g, b, m)
        o.backward(t["do"].double())
        out = dict(o=o.detach(), dq=q.grad, dk=k.grad, dv=v.grad)
        if b is not None:
            out["dbias"] = b.grad
        if g is not None:
            out["dscale"] = g.grad
        arrays = {kk: vv.numpy().astype(np.float32) for kk, vv in out.items()}
        # float64 scalars that survive the float32 storage: per-tensor L2 norms
        for kk, vv in out.items():
            arrays[kk + "_norm64"] = np.array(float(vv.double().norm()))
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(name, {kk: tuple(vv.shape) for kk, vv in out.items()}, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
