"""Seeded synthetic window-attention workloads.

The reference benchmarks on random tensors (benchmark/bench_attn.py:20-30) and
ships no dataset, so these generators ARE the workload.  Shapes and value
distributions follow the five benchmark configurations this repository is
measured on; the draw order is fixed (q, k, v, bias, upstream grad) so that a
seed reproduces the same tensors everywhere.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    """One window-attention problem: `batch` images of `nw` windows each."""
    name: str
    batch: int
    nw: int          # windows per image (mask.shape[0])
    heads: int
    window: int      # window side; N = window * window tokens
    head_dim: int = 32
    dtype: str = "bf16"   # "fp32" (oracle only), "fp16", "bf16"
    shift: int | None = None  # default window // 2

    @property
    def n(self) -> int:
        return self.window * self.window

    @property
    def bw(self) -> int:
        return self.batch * self.nw

    @property
    def units(self) -> int:
        """(window, head) pairs: the independent units of the hot path."""
        return self.bw * self.heads

    @property
    def map_side(self) -> int:
        return int(round(math.sqrt(self.nw))) * self.window

    def matmul_flops(self, fwd: bool = True, bwd: bool = True) -> float:
        """Matmul FLOPs only: forward 4*N^2*d, backward 10*N^2*d per unit."""
        per = (4 if fwd else 0) + (10 if bwd else 0)
        return float(per) * self.n * self.n * self.head_dim * self.units

    def algorithmic_bytes(self, fwd: bool = True, bwd: bool = True) -> float:
        """Unavoidable HBM traffic: forward reads q,k,v and writes o,lse; backward
        reads q,k,v,o,do,lse and writes dq,dk,dv; tables counted once per call."""
        e = 4 if self.dtype == "fp32" else 2
        n, d, u = self.n, self.head_dim, self.units
        tables = (self.heads + self.nw) * n * n * e
        total = 0.0
        if fwd:
            total += u * (4 * n * d * e + 4 * n) + tables
        if bwd:
            total += u * (8 * n * d * e + 4 * n) + tables + self.heads * n * n * e
        return total


# The five configurations the implementation is checked and measured on.
CONFIGS = {
    "cfg1": Workload("cfg1", batch=2, nw=4, heads=3, window=8, dtype="fp32"),
    "cfg2": Workload("cfg2", batch=64, nw=64, heads=3, window=8, dtype="fp16"),
    "cfg3": Workload("cfg3", batch=16, nw=16, heads=6, window=16, dtype="bf16"),
    "cfg4": Workload("cfg4", batch=64, nw=64, heads=3, window=16, dtype="bf16"),
}


def sweep(window: int) -> Workload:
    """TFLOPS sweep point: batch 16, 16 windows, 6 heads, d 32 (benchmark/config.py:4)."""
    return Workload(f"sweep_w{window}", batch=16, nw=16, heads=6, window=window, dtype="bf16")


TORCH_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def shift_mask(map_side: int, window: int, shift: int) -> torch.Tensor:
    """(nW,N,N) fp32 mask with 0 / -100, built the way a shifted Swin block does
    (flash_win_attn_v2/swin_transformer_v2.py:386-405)."""
    img = torch.zeros(map_side, map_side)
    bounds = (slice(0, -window), slice(-window, -shift), slice(-shift, None))
    region = 0
    for hs in bounds:
        for ws in bounds:
            img[hs, ws] = region
            region += 1
    g = map_side // window
    ids = img.reshape(g, window, g, window).permute(0, 2, 1, 3).reshape(g * g, window * window)
    diff = ids[:, None, :] - ids[:, :, None]
    return torch.where(diff != 0, torch.tensor(-100.0), torch.tensor(0.0))


def make_inputs(w: Workload, seed: int = 0, device="cpu", batch: int | None = None,
                with_mask: bool = True, with_bias: bool = True, with_scale: bool = True,
                logit_scale_value: float = math.log(10.0)):
    """Returns dict(q,k,v,bias,mask,logit_scale,do) in the workload dtype.

    Values are drawn in fp32 on the CPU generator (q, k, v, bias, do in that
    order) and then cast, so an fp32 oracle fed `x.float()` sees exactly the
    rounded inputs the kernels see.  `batch` overrides the image count (used for
    bounded CPU samples and per-rank shards).
    """
    b = w.batch if batch is None else batch
    gen = torch.Generator(device="cpu").manual_seed(seed)
    dt = TORCH_DTYPES[w.dtype]
    shape = (b * w.nw, w.heads, w.n, w.head_dim)
    q = torch.randn(shape, generator=gen)
    k = torch.randn(shape, generator=gen)
    v = torch.randn(shape, generator=gen)
    bias = 16.0 * torch.sigmoid(torch.randn(w.heads, w.n, w.n, generator=gen))
    do = torch.randn(shape, generator=gen)
    out = dict(q=q.to(dt), k=k.to(dt), v=v.to(dt), do=do.to(dt))
    out["bias"] = bias.to(dt) if with_bias else None
    if with_mask:
        shift = w.shift if w.shift is not None else w.window // 2
        out["mask"] = shift_mask(w.map_side, w.window, shift).to(dt)
    else:
        out["mask"] = None
    out["logit_scale"] = (torch.full((w.heads, 1, 1), logit_scale_value).to(dt)
                          if with_scale else None)
    if device != "cpu":
        out = {k_: (t.to(device) if t is not None else None) for k_, t in out.items()}
    return out


def make_reference_recipe_inputs(w: Workload, seed: int = 0, device="cpu"):
    """Inputs drawn the way the reference's own attention benchmark draws them
    (benchmark/bench_attn.py:20-30): q, k, v, bias and logit_scale ~ N(0, 1), a mask that is -inf
    where an independent N(0, 1) draw is negative and 0 elsewhere, and an upstream gradient of -1
    everywhere (its loss is `-out.sum()`).  Same dict as `make_inputs`."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    dt = TORCH_DTYPES[w.dtype]
    shape = (w.bw, w.heads, w.n, w.head_dim)
    out = {name: torch.randn(shape, generator=gen).to(dt) for name in ("q", "k", "v")}
    out["bias"] = torch.randn(w.heads, w.n, w.n, generator=gen).to(dt)
    draw = torch.randn(w.nw, w.n, w.n, generator=gen)
    out["mask"] = torch.zeros(w.nw, w.n, w.n).masked_fill(draw < 0, float("-inf")).to(dt)
    out["logit_scale"] = torch.randn(w.heads, 1, 1, generator=gen).to(dt)
    out["do"] = torch.full(shape, -1.0).to(dt)
    if device != "cpu":
        out = {k_: t.to(device) for k_, t in out.items()}
    return out
