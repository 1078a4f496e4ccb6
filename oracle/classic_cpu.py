"""Multi-threaded CPU port of the reference's classic window-attention path, forward + backward.

TEST / BASELINE INFRASTRUCTURE ONLY: used as the timed CPU baseline of the benchmark and by the
multi-process host-logic tests; never imported by the shipped package.

Same arithmetic as `oracle/window_attention_oracle.py` (which is pinned against golden vectors
of the reference, flash_win_attn_v2/win_attention_func.py:11-39), written with torch CPU
tensor ops so that it uses every host core the way the reference's PyTorch path would: fp32,
materialising the (BW, H, N, N) score tensor, explicit gradients instead of autograd.
"""
from __future__ import annotations

import math

import torch

LN_100 = math.log(100.0)


def forward_backward(q, k, v, do, logit_scale=None, bias=None, mask=None, with_magnitude=False):
    """fp32 CPU tensors in, dict(o, lse, dq, dk, dv, dbias, dscale) out.

    with_magnitude: also return `dscale_mag`, the per-head sum of the ABSOLUTE values of the terms
    dLogitScale adds up (the yardstick for its error when the signed sum nearly cancels)."""
    bw, h, n, d = q.shape
    qn = q.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    kn = k.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    qh, kh = q / qn, k / kn
    c = qh @ kh.transpose(-1, -2)
    if logit_scale is not None:
        s = logit_scale.reshape(1, h, 1, 1).clamp(max=LN_100).exp()
    else:
        s = torch.full((1, h, 1, 1), 1.0 / math.sqrt(d), dtype=q.dtype)
    a = c * s
    if bias is not None:
        a = a + bias.unsqueeze(0)
    if mask is not None:
        nw = mask.shape[0]
        a = (a.view(bw // nw, nw, h, n, n) + mask.unsqueeze(1).unsqueeze(0)).view(bw, h, n, n)
    lse = torch.logsumexp(a, dim=-1)
    p = torch.exp(a - lse.unsqueeze(-1))
    o = p @ v
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    delta = (do * o).sum(-1, keepdim=True)
    ds = p * (dp - delta)
    dbias = ds.sum(0) if bias is not None else None
    dc = ds * s
    dscale = dscale_mag = None
    if logit_scale is not None:
        gate = (logit_scale.reshape(h) <= LN_100).to(q.dtype)
        dscale = ((dc * c).sum(dim=(0, 2, 3)) * gate).reshape(h, 1, 1)
        if with_magnitude:
            dscale_mag = (dc * c).abs().sum(dim=(0, 2, 3))
    dqh = dc @ kh
    dkh = dc.transpose(-1, -2) @ qh
    dq = (dqh - qh * (qh * dqh).sum(-1, keepdim=True)) / qn
    dk = (dkh - kh * (kh * dkh).sum(-1, keepdim=True)) / kn
    return dict(o=o, lse=lse, dq=dq, dk=dk, dv=dv, dbias=dbias, dscale=dscale, dscale_mag=dscale_mag)
