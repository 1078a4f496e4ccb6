"""Host logic of the window-sharded multi-GPU path, on CPU ranks (gloo, world size 2).

The per-rank compute is replaced by the CPU oracle; what is tested is the partition on image
boundaries, the packed fp32 [dBias | dLogitScale] all-reduce and the finalisation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_window_attention_v2_b200 import sharded
from flash_window_attention_v2_b200.workloads import Workload, make_inputs
from oracle import classic_cpu
from oracle import window_attention_oracle as orc


def test_image_ranges_cover_everything():
    for batch in (1, 7, 8, 64):
        for world in (1, 2, 3, 8):
            got = []
            for r in range(world):
                s, c = sharded.image_range(batch, world, r)
                got += list(range(s, s + c))
            assert got == list(range(batch))
    sl = sharded.window_slice(8, 16, 4, 1)
    assert (sl.start, sl.stop) == (32, 64)
    with pytest.raises(ValueError):
        sharded.image_range(4, 2, 2)


class OracleBackend:
    """CPU stand-in for the CUDA kernels with the same three-step interface."""

    @staticmethod
    def forward(q, k, v, ls, bias, mask, scale_type):
        return None, None, ls

    @staticmethod
    def backward_partial(do, q, k, v, ls, o, lse, bias, mask, scale_type):
        r = classic_cpu.forward_backward(q, k, v, do, ls if scale_type == "tensor" else None, bias, mask)
        h, n = q.shape[1], q.shape[2]
        partial = torch.zeros(h * n * n + h)
        if bias is not None:
            partial[: h * n * n] = r["dbias"].reshape(-1)
        if scale_type == "tensor":
            # before the clamp gate, as the CUDA path leaves it
            c = torch.nn.functional.normalize(q, dim=-1) @ torch.nn.functional.normalize(k, dim=-1).transpose(-1, -2)
            s = ls.reshape(1, h, 1, 1).clamp(max=classic_cpu.LN_100).exp()
            a = c * s + (bias.unsqueeze(0) if bias is not None else 0)
            if mask is not None:
                nw = mask.shape[0]
                a = (a.view(-1, nw, h, n, n) + mask[None, :, None]).view(-1, h, n, n)
            p = torch.softmax(a, -1)
            dp = do @ v.transpose(-1, -2)
            ds = p * (dp - (p * dp).sum(-1, keepdim=True))
            partial[h * n * n:] = (ds * s * c).sum(dim=(0, 2, 3))
        OracleBackend.last = r
        return r["dq"], r["dk"], r["dv"], partial

    @staticmethod
    def finalize(partial, ls, bias, scale_type):
        h, n = bias.shape[0], bias.shape[1]
        db = partial[: h * n * n].reshape(h, n, n).clone()
        gate = (ls.reshape(h) <= classic_cpu.LN_100).float()
        return db, (partial[h * n * n:] * gate).reshape(h, 1, 1)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    w = Workload("shard", batch=4, nw=4, heads=2, window=8, dtype="fp32")
    t = make_inputs(w, seed=0)
    t["logit_scale"][1] = 5.0   # one clamped head: its gradient must come out as zero
    sl = sharded.window_slice(w.batch, w.nw, world, rank)
    o, dq, dk, dv, dscale, db = sharded.sharded_step(
        OracleBackend, dist.group.WORLD, t["q"][sl], t["k"][sl], t["v"][sl], t["do"][sl],
        t["logit_scale"], t["bias"], t["mask"])
    full = classic_cpu.forward_backward(t["q"], t["k"], t["v"], t["do"], t["logit_scale"], t["bias"], t["mask"])
    res = dict(
        dq=orc.rel_err(dq.numpy(), full["dq"][sl].numpy()),
        dk=orc.rel_err(dk.numpy(), full["dk"][sl].numpy()),
        db=orc.rel_err(db.numpy(), full["dbias"].numpy()),
        dscale=float((dscale - full["dscale"]).abs().max() / full["dscale"].abs().max()),
        clamped_zero=float(dscale[1].abs().max()),
    )
    out[rank] = res
    dist.destroy_process_group()


def test_two_rank_sharded_step_matches_unsharded():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
        assert set(out.keys()) == {0, 1}
        for r in out.values():
            assert r["dq"] < 1e-5 and r["dk"] < 1e-5
            assert r["db"] < 1e-5
            assert r["dscale"] < 1e-4
            assert r["clamped_zero"] == 0.0
