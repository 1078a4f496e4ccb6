"""Forward + backward for batches that live in HOST memory.

A caller whose activations sit in pinned host buffers (an offloading trainer, a plugin boundary that
hands over host pointers) pays for two PCIe transfers per batch that are each ten times longer
than the kernels.  `HostBatchPipeline` overlaps the three stages of consecutive batches on three
CUDA streams -- host->device copy of batch i+1, kernels of batch i, device->host copy of the
results of batch i-1 -- with double-buffered device inputs, so that the throughput is set by the
slower PCIe direction instead of by the sum of all three.

Nothing here computes on the host: the work is done by `flash_win_attn_v2_func` and autograd.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .flash_window_attention_v2 import flash_win_attn_v2_func

_INPUT_KEYS = ("q", "k", "v", "do", "logit_scale", "bias", "mask")


class HostBatchPipeline:
    """submit(host_batch, host_out) enqueues one batch and returns at once; drain() waits for all.

    host_batch: dict with pinned CPU tensors q, k, v, do (BW, H, N, d), logit_scale (H, 1, 1),
    bias (H, N, N) and mask (nW, N, N) (the last three may be None).
    host_out: list of pinned CPU tensors that receive (o, dq, dk, dv[, dlogit_scale][, dbias]), or
    None to let the pipeline allocate them (returned by submit()).
    """

    def __init__(self, device: torch.device, depth: int = 2, attn_func=flash_win_attn_v2_func):
        assert depth >= 2
        self.device = device
        self.attn_func = attn_func   # same signature as flash_win_attn_v2_func (e.g. the sharded one)
        self.depth = depth
        self.s_in = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self._slots: List[Optional[Dict[str, Optional[torch.Tensor]]]] = [None] * depth
        self._slot_free = [None] * depth      # event: kernels that read the slot have finished
        self._out_done = [None] * depth       # event: the results of the slot have reached the host
        self._host_out: List[Optional[List[torch.Tensor]]] = [None] * depth
        self._n = 0

    def _device_slot(self, i: int, host_batch) -> Dict[str, Optional[torch.Tensor]]:
        slot = self._slots[i]
        if slot is None:
            slot = {k: (torch.empty(v.shape, dtype=v.dtype, device=self.device) if v is not None else None)
                    for k, v in host_batch.items() if k in _INPUT_KEYS}
            self._slots[i] = slot
        return slot

    def submit(self, host_batch, host_out: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        i = self._n % self.depth
        self._n += 1
        compute = torch.cuda.current_stream(self.device)
        slot = self._device_slot(i, host_batch)

        # ---- stage 1: host -> device, as soon as the kernels of the batch before last are done
        with torch.cuda.stream(self.s_in):
            if self._slot_free[i] is not None:
                self.s_in.wait_event(self._slot_free[i])
            for k, dst in slot.items():
                if dst is not None:
                    dst.copy_(host_batch[k], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(self.s_in)

        # ---- stage 2: kernels
        compute.wait_event(ev_in)
        q, k_, v = (slot[x].detach().requires_grad_(True) for x in ("q", "k", "v"))
        wrt = [q, k_, v]
        ls = slot.get("logit_scale")
        bias = slot.get("bias")
        if ls is not None:
            ls = ls.detach().requires_grad_(True)
            wrt.append(ls)
        if bias is not None:
            bias = bias.detach().requires_grad_(True)
            wrt.append(bias)
        o = self.attn_func(q, k_, v, ls, bias, slot.get("mask"))
        results = [o.detach()] + list(torch.autograd.grad(o, wrt, slot["do"]))
        ev_done = torch.cuda.Event()
        ev_done.record(compute)
        self._slot_free[i] = ev_done

        # ---- stage 3: device -> host
        if host_out is None:
            if self._host_out[i] is None:
                self._host_out[i] = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in results]
            host_out = self._host_out[i]
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(ev_done)
            for hbuf, r in zip(host_out, results):
                r.record_stream(self.s_out)
                hbuf.copy_(r, non_blocking=True)
            ev_out = torch.cuda.Event()
            ev_out.record(self.s_out)
        self._out_done[i] = ev_out
        return list(host_out)

    def drain(self) -> None:
        self.s_in.synchronize()
        torch.cuda.current_stream(self.device).synchronize()
        self.s_out.synchronize()
        # everything has finished: a device-side timeout of any submitted batch is visible now
        from . import kernels
        kernels.poll_device_status(self.device)
