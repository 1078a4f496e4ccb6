"""Forward + backward captured once into a CUDA graph and replayed.

One training step of this op is four short kernels (forward; table transpose, backward, dBias
reduction) whose device time at small windows is comparable to the time the host needs to get
through autograd and the argument marshalling.  Capturing the step removes the host from the loop:
`GraphedStep` owns static input and output tensors, `replay()` relaunches the recorded kernels.

The captured work is exactly `flash_win_attn_v2_func` followed by `torch.autograd.grad`; the tensor
maps inside the library calls are encoded at capture time for the static buffers.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import kernels as _kernels
from .flash_window_attention_v2 import flash_win_attn_v2_func


class GraphedStep:
    """Static-buffer fwd + bwd.  Fill `.q .k .v .do` (and `.logit_scale .bias .mask`) in place,
    call `replay()`, read `.outputs` = [o, dq, dk, dv(, dlogit_scale)(, dbias)]."""

    def __init__(self, q, k, v, do, logit_scale=None, bias=None, mask=None, attn_func=flash_win_attn_v2_func):
        dev = q.device
        self.q, self.k, self.v = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
        self.do = do.detach().clone()
        self.logit_scale = logit_scale.detach().clone().requires_grad_(True) if logit_scale is not None else None
        self.bias = bias.detach().clone().requires_grad_(True) if bias is not None else None
        self.mask = mask.detach().clone() if mask is not None else None
        wrt = [self.q, self.k, self.v]
        if self.logit_scale is not None:
            wrt.append(self.logit_scale)
        if self.bias is not None:
            wrt.append(self.bias)

        def step() -> List[torch.Tensor]:
            o = attn_func(self.q, self.k, self.v, self.logit_scale, self.bias, self.mask)
            return [o.detach()] + list(torch.autograd.grad(o, wrt, self.do))

        # warm up on a side stream (library initialisation, allocator), then capture
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.outputs: List[torch.Tensor] = step()

    def replay(self) -> List[torch.Tensor]:
        # a device-side timeout of an earlier replay shows up here (host read of a pinned word)
        _kernels.poll_device_status(self.q.device)
        self.graph.replay()
        return self.outputs
