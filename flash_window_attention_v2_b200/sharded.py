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
import os
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


class PeerReducer:
    """The cross-GPU sum of dBias / dLogitScale as ONE kernel per GPU over peer memory
    (`fwa2_peer_reduce_finalize`): every rank's fp32 sums live in symmetric memory that all ranks
    have mapped; the kernel exchanges one flag per peer, adds the buffers in rank order and casts.
    Two buffer sets alternate from call to call (a fast rank may start the next step while a slow
    one still reads this step's sums).  Raises at construction if symmetric memory is unavailable;
    callers then stay on the NCCL all-reduce."""

    def __init__(self, heads: int, n: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        import ctypes as C

        import torch.distributed._symmetric_memory as symm
        self._C = C
        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise RuntimeError("fwa2_peer_reduce_finalize is built for at most 8 peers")
        self.heads, self.n = heads, n
        numel = heads * n * n + heads
        self.bufs = [symm.empty(numel, dtype=torch.float32, device=device) for _ in range(2)]
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.flags.zero_()
        for b in self.bufs:
            b.zero_()
        torch.cuda.synchronize(device)
        name = group.group_name
        self._hdls = [symm.rendezvous(b, name) for b in self.bufs]
        self._hflag = symm.rendezvous(self.flags, name)
        self._buf_ptrs = [(C.c_void_p * self.world)(*[int(p) for p in h.buffer_ptrs]) for h in self._hdls]
        self._flag_ptrs = (C.c_void_p * self.world)(*[int(p) for p in self._hflag.buffer_ptrs])
        self._hflag.barrier()          # every rank's flags are zero before anybody writes one
        self.epoch = 0

    def next_buffer(self) -> torch.Tensor:
        """The buffer the NEXT call of reduce() will read on this rank: hand it to the backward as
        its `_partial_out`."""
        return self.bufs[(self.epoch + 1) & 1]

    def reduce(self, logit_scale, db, dscale) -> None:
        """Sum over the ranks and cast into db / dscale (either may be None).  Stream-ordered after
        the backward that filled next_buffer(); returns at once."""
        from . import _lib, kernels
        self.epoch += 1
        ref = db if db is not None else dscale
        with torch.cuda.device(ref.device):
            _lib.check(_lib.lib().fwa2_peer_reduce_finalize(
                self._buf_ptrs[self.epoch & 1], self._flag_ptrs, self.rank, self.world, self.epoch & 0xFFFFFFFF,
                kernels._DTYPES[ref.dtype], self.heads, self.n,
                logit_scale.data_ptr() if dscale is not None else None,
                db.data_ptr() if db is not None else None, dscale.data_ptr() if dscale is not None else None,
                kernels._status(ref.device).data_ptr(),
                self._C.c_void_p(torch.cuda.current_stream(ref.device).cuda_stream)), "fwa2_peer_reduce_finalize")


class GraphedShardedStep:
    """Forward + backward of this rank's windows with the local kernels captured in CUDA graphs.

    The graph holds what needs no other rank (forward, backward, the local fp32 sums of dBias and
    dLogitScale); the exchange step runs outside it, so that nothing that can block on a peer is
    inside a capture: with a `PeerReducer` one fused kernel over peer memory (two graphs, one per
    buffer set, replayed alternately), otherwise one NCCL all-reduce of `H*N*N + H` floats and the
    cast kernel.  Fill `.q .k .v .do` in place, call `replay()`, read
    `(o, dq, dk, dv, dscale, dbias)`."""

    def __init__(self, q, k, v, do, logit_scale, bias, mask, group: Optional[dist.ProcessGroup] = None,
                 reducer: Optional[PeerReducer] = None):
        dev = q.device
        self.group = group
        self.reducer = reducer
        self.q, self.k, self.v, self.do = (x.detach().clone() for x in (q, k, v, do))
        self.logit_scale = logit_scale.detach().clone() if logit_scale is not None else None
        self.bias = bias.detach().clone() if bias is not None else None
        self.mask = mask.detach().clone() if mask is not None else None
        if self.logit_scale is not None:
            self.scale_type, self._ls = "tensor", self.logit_scale
        else:
            self.scale_type = "scalar"
            self._ls = torch.tensor(1.0 / math.sqrt(q.shape[-1]), device=dev)
        self._need = self.bias is not None or self.scale_type == "tensor"

        def local(partial):
            from . import kernels
            o, lse, ls = CudaBackend.forward(self.q, self.k, self.v, self._ls, self.bias, self.mask, self.scale_type)
            dq, dk, dv = torch.empty_like(self.q), torch.empty_like(self.k), torch.empty_like(self.v)
            kernels._flash_attn_backward(self.do, self.q, self.k, self.v, ls, o, lse, dq, dk, dv, None, None,
                                         bias=self.bias, mask=self.mask, scale_type=self.scale_type,
                                         _partial_out=partial)
            return o, dq, dk, dv

        h, n = q.shape[1], q.shape[2]
        if reducer is not None and self._need:
            partials = list(reducer.bufs)
        elif self._need:
            partials = [torch.zeros(h * n * n + h, dtype=torch.float32, device=dev)]
        else:
            partials = [None]
        self._partials = partials
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            scratch = torch.zeros(h * n * n + h, dtype=torch.float32, device=dev) if self._need else None
            for _ in range(2):
                local(scratch)       # warm-up must not touch buffers that peers may be reading
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graphs, self.outs = [], []
        for pbuf in partials:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.outs.append(local(pbuf))
            self.graphs.append(g)
        self.db = torch.empty_like(self.bias) if self.bias is not None else None
        self.dscale = torch.empty_like(self.logit_scale) if self.scale_type == "tensor" else None

    def replay(self):
        from . import kernels
        kernels.poll_device_status(self.q.device)
        if self.reducer is not None and self._need:
            i = (self.reducer.epoch + 1) & 1
            self.graphs[i].replay()
            self.reducer.reduce(self._ls, self.db, self.dscale)
            o, dq, dk, dv = self.outs[i]
            return o, dq, dk, dv, self.dscale, self.db
        self.graphs[0].replay()
        o, dq, dk, dv = self.outs[0]
        db = dscale = None
        if self._need:
            partial = self._partials[0]
            if self.group is not None or (dist.is_initialized() and dist.get_world_size() > 1):
                dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
            kernels.finalize_grads(partial, self._ls, self.db, self.dscale)
            db, dscale = self.db, self.dscale
        return o, dq, dk, dv, dscale, db


def sharded_parity_check(w, device, reducer: Optional[PeerReducer] = None, images_per_rank: int = 1):
    """Before a multi-GPU measurement: a small problem that every rank holds in full (same seed),
    computed unsharded on this GPU with the plain function and sharded over the ranks; this rank's
    slice of o / dq / dk / dv must agree bitwise (a window's results do not depend on which other
    windows share the launch) and the summed dBias / dLogitScale to rounding.  Returns a dict with
    the worst deviations over all ranks."""
    from .flash_window_attention_v2 import flash_win_attn_v2_func
    from .workloads import Workload, make_inputs
    world, rank = dist.get_world_size(), dist.get_rank()
    small = Workload(w.name + "_parity", batch=images_per_rank * world, nw=w.nw, heads=w.heads, window=w.window,
                     dtype=w.dtype)
    t = make_inputs(small, seed=1234, device=device)
    q, k, v = (t[x].detach().requires_grad_(True) for x in ("q", "k", "v"))
    ls, bias = t["logit_scale"].detach().requires_grad_(True), t["bias"].detach().requires_grad_(True)
    o = flash_win_attn_v2_func(q, k, v, ls, bias, t["mask"])
    ref = (o,) + torch.autograd.grad(o, (q, k, v, ls, bias), t["do"])
    sl = window_slice(small.batch, small.nw, world, rank)
    step = GraphedShardedStep(t["q"][sl], t["k"][sl], t["v"][sl], t["do"][sl], t["logit_scale"], t["bias"], t["mask"],
                              reducer=reducer)
    so, sdq, sdk, sdv, sds, sdb = step.replay()
    torch.cuda.synchronize(device)
    rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))
    # worst absolute deviation of this rank's o / dq / dk / dv from the unsharded run (0 = bitwise equal)
    worst = [float((a.float() - b[sl].float()).abs().max()) for a, b in zip((so, sdq, sdk, sdv), ref[:4])]
    exact = all(torch.equal(a, b[sl]) for a, b in zip((so, sdq, sdk, sdv), ref[:4]))
    dev_db, dev_ds = rel(sdb, ref[5]), rel(sds, ref[4])
    stats = torch.tensor([0.0 if exact else 1.0, dev_db, dev_ds] + worst, device=device)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    # every rank must also hold the SAME summed gradients, bit for bit
    mine = torch.cat([sdb.float().reshape(-1), sds.float().reshape(-1)])
    lo, hi = mine.clone(), mine.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return dict(images=small.batch, window_results_bitwise_equal=bool(stats[0].item() == 0.0),
                max_abs_dev_o_dq_dk_dv=[float(x) for x in stats[3:7]],
                dbias_rel_dev=float(stats[1]), dscale_rel_dev=float(stats[2]),
                sums_identical_on_all_ranks=bool(torch.equal(lo, hi)))


def make_sharded_step(t, w, device, kernels_module=None):
    """What bench.py times on N > 1 GPUs: this rank's share of the images, local kernels replayed
    from CUDA graphs, then the cross-GPU sum of dBias / dLogitScale -- the fused peer-memory kernel
    when symmetric memory can be set up, the NCCL all-reduce otherwise.  Returns
    (step, parity_report, description)."""
    reducer = None
    why = ""
    if os.environ.get("FWA2_SHARDED_EXCHANGE", "peer") == "peer":
        try:
            reducer = PeerReducer(t["q"].shape[1], t["q"].shape[2], device)
        except Exception as ex:      # no symmetric memory on this system: say so, use NCCL
            why = f" (peer-memory exchange unavailable: {type(ex).__name__}: {ex})"
    parity = sharded_parity_check(w, device, reducer)
    step = GraphedShardedStep(t["q"], t["k"], t["v"], t["do"], t["logit_scale"], t["bias"], t["mask"], reducer=reducer)
    api = ("GraphedShardedStep: local kernels replayed from a CUDA graph, then " +
           ("one fused peer-memory kernel (fwa2_peer_reduce_finalize over NVLink) for the sum of dBias / dLogitScale"
            if reducer is not None else "NCCL all-reduce + cast of dBias / dLogitScale" + why))
    return step.replay, parity, api
