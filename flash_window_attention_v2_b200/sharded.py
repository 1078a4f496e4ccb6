"""Window-sharded multi-GPU window attention (one process per GPU).

Units (window, head) are independent in the forward pass and for dQ, dK, dV, so the
`batch * n_windows` axis is split across ranks on IMAGE boundaries (a rank's slice is a multiple
of `n_windows`, which keeps `local_row mod n_windows` selecting the right mask).  Bias, mask and
logit_scale are replicated.  The only exchange step is the sum of dBias (H, N, N) and
dLogitScale (H) over all windows: each rank reduces its own windows into ONE packed fp32 buffer
`[H*N*N | H]`, the buffer is all-reduced (NCCL over NVLink on GPUs), and every rank then applies
the clamp gate and casts once, exactly as the single-GPU path does.

Under DistributedDataParallel this module is NOT what you want: there every replica keeps its
own bias gradient and DDP averages parameter gradients; use the plain function.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist


def image_range(batch: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced split of `batch` images: (first image, number of images)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank / world size")
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def window_slice(batch: int, n_windows: int, world: int, rank: int) -> slice:
    """Rows of the (batch * n_windows) axis owned by `rank`."""
    start, count = image_range(batch, world, rank)
    return slice(start * n_windows, (start + count) * n_windows)


class CudaBackend:
    """The sm_100a kernels behind the three steps of the sharded backward."""

    @staticmethod
    def forward(q, k, v, logit_scale, bias, mask, scale_type):
        from . import kernels
        return kernels._flash_attn_forward(q, k, v, logit_scale, bias=bias, mask=mask, scale_type=scale_type)

    @staticmethod
    def backward_partial(do, q, k, v, logit_scale, o, lse, bias, mask, scale_type):
        """Returns (dq, dk, dv, partial) with partial = fp32 [H*N*N | H] local sums (or None)."""
        from . import kernels
        h, n = q.shape[1], q.shape[2]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        need = bias is not None or scale_type == "tensor"
        partial = torch.zeros(h * n * n + h, dtype=torch.float32, device=q.device) if need else None
        kernels._flash_attn_backward(do, q, k, v, logit_scale, o, lse, dq, dk, dv, None, None,
                                     bias=bias, mask=mask, scale_type=scale_type, _partial_out=partial)
        return dq, dk, dv, partial

    @staticmethod
    def finalize(partial, logit_scale, bias, scale_type):
        from . import kernels
        db = torch.empty_like(bias) if bias is not None else None
        dscale = torch.empty_like(logit_scale) if scale_type == "tensor" else None
        kernels.finalize_grads(partial, logit_scale, db, dscale)
        return db, dscale


def sharded_step(backend, group, q, k, v, do, logit_scale, bias, mask):
    """Forward + backward of this rank's windows with the cross-rank gradient sum.

    Returns (o, dq, dk, dv, dscale, dbias).  `backend` supplies the per-rank compute (the CUDA
    kernels in production, a CPU stand-in in the host-logic tests)."""
    if logit_scale is not None:
        scale_type, ls = "tensor", logit_scale
    else:
        scale_type = "scalar"
        ls = torch.tensor(1.0 / math.sqrt(q.shape[-1]), device=q.device)
    o, lse, ls = backend.forward(q, k, v, ls, bias, mask, scale_type)
    dq, dk, dv, partial = backend.backward_partial(do, q, k, v, ls, o, lse, bias, mask, scale_type)
    db = dscale = None
    if partial is not None:
        if group is not None and dist.get_world_size(group) > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
        db, dscale = backend.finalize(partial, ls, bias, scale_type)
    return o, dq, dk, dv, dscale, db


class ShardedFlashWindowAttentionV2(torch.autograd.Function):
    """Autograd Function over a rank's LOCAL windows; dBias / dLogitScale are summed over the
    process group in backward.  Same argument order as the single-GPU Function, plus `group`."""

    @staticmethod
    def forward(ctx, q, k, v, logit_scale=None, bias=None, mask=None, group=None):
        if logit_scale is not None:
            scale_type, ls = "tensor", (logit_scale if logit_scale.stride(-1) == 1 else logit_scale.contiguous())
        else:
            scale_type = "scalar"
            ls = torch.tensor(1.0 / math.sqrt(q.shape[-1]), device=q.device)
        q, k, v = [x if x.stride(-1) == 1 else x.contiguous() for x in (q, k, v)]
        o, lse, ls = CudaBackend.forward(q, k, v, ls, bias, mask, scale_type)
        ctx.save_for_backward(q, k, v, o, lse, ls, bias, mask)
        ctx.scale_type = scale_type
        ctx.group = group
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, ls, bias, mask = ctx.saved_tensors
        dq, dk, dv, partial = CudaBackend.backward_partial(do, q, k, v, ls, o, lse, bias, mask, ctx.scale_type)
        db = dscale = None
        if partial is not None:
            if ctx.group is not None or (dist.is_initialized() and dist.get_world_size() > 1):
                dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=ctx.group)
            db, dscale = CudaBackend.finalize(partial, ls, bias, ctx.scale_type)
        return dq, dk, dv, dscale, db, None, None


def sharded_flash_win_attn_v2_func(q, k, v, logit_scale=None, bias=None, mask=None,
                                   group: Optional[dist.ProcessGroup] = None):
    return ShardedFlashWindowAttentionV2.apply(q, k, v, logit_scale, bias, mask, group)


class GraphedShardedStep:
    """Forward + backward of this rank's windows with the local kernels captured in a CUDA graph.

    The graph holds what needs no other rank (forward, backward, the local fp32 sums of dBias and
    dLogitScale); the exchange step -- one NCCL all-reduce of `H*N*N + H` floats -- and the final
    cast run outside it, so that nothing that can block on a peer is inside a capture.
    Fill `.q .k .v .do` in place, call `replay()`, read `(o, dq, dk, dv, dscale, dbias)`."""

    def __init__(self, q, k, v, do, logit_scale, bias, mask, group: Optional[dist.ProcessGroup] = None):
        dev = q.device
        self.group = group
        self.q, self.k, self.v, self.do = (x.detach().clone() for x in (q, k, v, do))
        self.logit_scale = logit_scale.detach().clone() if logit_scale is not None else None
        self.bias = bias.detach().clone() if bias is not None else None
        self.mask = mask.detach().clone() if mask is not None else None
        if self.logit_scale is not None:
            self.scale_type, self._ls = "tensor", self.logit_scale
        else:
            self.scale_type = "scalar"
            self._ls = torch.tensor(1.0 / math.sqrt(q.shape[-1]), device=dev)

        def local():
            o, lse, ls = CudaBackend.forward(self.q, self.k, self.v, self._ls, self.bias, self.mask, self.scale_type)
            dq, dk, dv, partial = CudaBackend.backward_partial(self.do, self.q, self.k, self.v, ls, o, lse,
                                                               self.bias, self.mask, self.scale_type)
            return o, dq, dk, dv, partial

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                local()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.o, self.dq, self.dk, self.dv, self.partial = local()

    def replay(self):
        from . import kernels
        kernels.poll_device_status(self.q.device)
        self.graph.replay()
        db = dscale = None
        if self.partial is not None:
            if self.group is not None or (dist.is_initialized() and dist.get_world_size() > 1):
                dist.all_reduce(self.partial, op=dist.ReduceOp.SUM, group=self.group)
            db, dscale = CudaBackend.finalize(self.partial, self._ls, self.bias, self.scale_type)
        return self.o, self.dq, self.dk, self.dv, dscale, db
