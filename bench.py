#!/usr/bin/env python
"""Benchmark of the window-attention hot path: forward + backward TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config cfg4] [--impl ours|reference]

One "step" is one forward + backward pass of the op over the whole workload, through the public
autograd API (`flash_win_attn_v2_func` + `torch.autograd.grad`).  The default workload is cfg4:
Swin-V2 patch 2 / window 16 stage-1 attention on 64 images of 256 x 256 (4096 windows of 256
tokens, 3 heads, head dimension 32, bf16).  With N > 1 (launched by torch.distributed.run, one
rank per GPU) the 64 images are SHARDED over the ranks on image boundaries (strong scaling); the
only exchange step is the sum of dBias / dLogitScale inside backward.  Rank 0 prints ONE JSON line.

`--impl reference` times the reference's classic PyTorch path (`win_attention_torch` with
autograd, fp32) on the host CPU cores -- the installed reference itself when it is present under
baseline/_ref, its port in oracle/classic_cpu.py otherwise.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flash_window_attention_v2_b200.workloads import (CONFIGS, Workload, make_inputs,  # noqa: E402
                                                      make_reference_recipe_inputs, sweep)

METRIC = "fwd+bwd window-attention throughput (matmul FLOPs 14*N^2*d per window-head)"
UNIT = "TFLOP/s"
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel (the backward
# main kernel), from the ncu captures summarised in profiles/.  cfg4 was not captured itself (its
# working set is beyond what a full-metric capture should hold): it is the cfg3 figure times 8, the
# ratio of window-heads, the traffic of this kernel being proportional to them.
NCU_TRAFFIC = {"cfg2": 368.9e6, "cfg3": 176.9e6, "cfg4": 8 * 176.9e6}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks, power and throttle reasons while the timed region runs (read-only).

    NVML through pynvml when it is importable (a query takes well under a millisecond, so that
    even a timed region of a few milliseconds gets samples), nvidia-smi otherwise."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []      # (sm_mhz, sm_max_mhz, power_w, hw_slowdown, hw_thermal, sw_thermal, sw_power_cap)
        self.source = None
        self._stop = threading.Event()
        self._thread = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

    def _run_nvml(self):
        import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(self._physical_index())
        mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = dict(hw=0x8, hw_th=0x40, sw_th=0x20, sw_pw=0x4)   # NVML clocks event reason bits
        self.source = "nvml"
        while not self._stop.is_set():
            r = int(get_reasons(h))
            self.samples.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), mx,
                                 nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                                 bool(r & bits["hw"]), bool(r & bits["hw_th"]), bool(r & bits["sw_th"]),
                                 bool(r & bits["sw_pw"])))
            self._stop.wait(0.002)

    def _run_smi(self):
        self.source = "nvidia-smi"
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [x.strip() for x in out.stdout.strip().split(",")]
                if len(parts) >= 7:
                    self.samples.append((float(parts[0]), float(parts[1]), float(parts[2]),
                                         *(x.lower().startswith("active") for x in parts[3:7])))
            except Exception:
                pass
            self._stop.wait(0.05)

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(s[0] for s in self.samples)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [nme for i, nme in enumerate(names) if any(s[3 + i] for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.samples[0][1],
                "power_w_max": max(s[2] for s in self.samples), "samples": len(sm), "source": self.source,
                "reasons": reasons}


# ------------------------------------------------------------------------------------------------
# The CPU arm: the reference's classic path, fp32, on the host cores
# ------------------------------------------------------------------------------------------------
def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core it may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))


def classic_path():
    """(kind, function).  function(q, k, v, do, logit_scale, bias, mask) runs one forward + backward
    of the classic path in fp32 on CPU tensors and returns (dbias, dscale).  "reference": the
    installed reference's own `win_attention_torch` under autograd; "port": oracle/classic_cpu.py."""
    if os.path.isdir(os.path.join(REF_DIR, "flash_win_attn_v2")):
        try:
            # the classic path lives in win_attention_func.py; its Triton kernels are not needed, so
            # this library's boundary stands in for them and Triton is never imported
            from flash_window_attention_v2_b200 import install
            install()
            if REF_DIR not in sys.path:
                sys.path.insert(0, REF_DIR)
            from flash_win_attn_v2.win_attention_func import win_attention_torch

            def run(q, k, v, do, ls, bias, mask):
                q, k, v = (x.detach().requires_grad_(True) for x in (q, k, v))
                ls, bias = ls.detach().requires_grad_(True), bias.detach().requires_grad_(True)
                o = win_attention_torch(q, k, v, ls, bias, mask)
                g = torch.autograd.grad(o, (q, k, v, ls, bias), do)
                return g[4], g[3]
            return "reference", run
        except Exception as ex:      # fall back to the port, and say why
            print(f"bench: installed reference unusable ({type(ex).__name__}: {ex}); using the port", file=sys.stderr)
    from oracle import classic_cpu

    def run(q, k, v, do, ls, bias, mask):
        r = classic_cpu.forward_backward(q, k, v, do, ls, bias, mask)
        return r["dbias"], r["dscale"]
    return "port", run


def classic_step(run, f, w, images, chunk):
    """One pass of the classic path over `images` images of `w`, a few images at a time (the path
    materialises (BW, H, N, N) in fp32); dBias and dLogitScale are summed over the chunks."""
    db = ds = None
    for i0 in range(0, images, chunk):
        sel = slice(i0 * w.nw, min(images, i0 + chunk) * w.nw)
        b, s = run(f["q"][sel], f["k"][sel], f["v"][sel], f["do"][sel], f["logit_scale"], f["bias"], f["mask"])
        db = b if db is None else db + b
        ds = s if ds is None else ds + s
    return db, ds


def cpu_plan(w, run, f, steps_total, budget_s):
    """Images per step so that `steps_total` steps fit `budget_s`: the full workload when it fits."""
    chunk = max(1, int(2.0e8 // (w.nw * w.heads * w.n * w.n * 4)))
    t0 = time.perf_counter()
    classic_step(run, f, w, min(chunk, w.batch), chunk)        # also the warm-up of the thread pool
    t0 = time.perf_counter()
    classic_step(run, f, w, min(chunk, w.batch), chunk)
    per_image = (time.perf_counter() - t0) / min(chunk, w.batch)
    fit = int(budget_s / max(per_image * steps_total, 1e-9))
    images = w.batch if fit >= w.batch else max(chunk, (fit // chunk) * chunk)
    return min(images, w.batch), chunk, per_image


def host_inputs(w):
    t = make_inputs(w, seed=0)
    return {k: (v.float() if v is not None else None) for k, v in t.items()}


def cpu_baseline(w, seconds: float = 15.0):
    use_all_host_threads()
    kind, run = classic_path()
    f = host_inputs(w)
    images, chunk, _ = cpu_plan(w, run, f, 1, seconds)
    n, t0 = 0, time.perf_counter()
    while True:
        classic_step(run, f, w, images, chunk)
        n += 1
        el = time.perf_counter() - t0
        if el >= seconds * 0.6 or n >= 50:
            break
    flops = 14.0 * w.n * w.n * w.head_dim * images * w.nw * w.heads
    return dict(value=flops * n / el / 1e12, unit=UNIT, cores=torch.get_num_threads(), kind=kind,
                sample=f"{images} of {w.batch} images ({images * w.nw * w.heads} window-heads) per pass, "
                       f"{n} passes in {el:.1f} s, fp32, host cpu_count={os.cpu_count()}",
                seconds_per_full_step=el / n * w.batch / images)


def run_reference(args, w, rank):
    """The reference arm: the classic path on the host cores; rank 0 only."""
    if rank != 0:
        return
    use_all_host_threads()
    kind, run = classic_path()
    f = host_inputs(w)
    warm = max(1, min(args.warmup, 2))
    images, chunk, per_image = cpu_plan(w, run, f, args.steps + warm, 200.0)
    for _ in range(warm):
        classic_step(run, f, w, images, chunk)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        classic_step(run, f, w, images, chunk)
    el = time.perf_counter() - t0
    flops = 14.0 * w.n * w.n * w.head_dim * images * w.nw * w.heads
    val = flops * args.steps / el / 1e12
    sample = (f"each step = {images} of {w.batch} images ({images * w.nw * w.heads} window-heads) of {w.name}, "
              f"in chunks of {chunk} images with dBias / dLogitScale summed over the chunks; fp32 classic path "
              f"({'the installed reference' if kind == 'reference' else 'port of the reference'}) on host cores")
    line = dict(impl="reference", metric=METRIC, value=val, unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=warm, ms_per_step=el / args.steps * 1e3, higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=w.name, images_per_step=images, images=w.batch, windows_per_image=w.nw,
                            heads=w.heads, n=w.n, head_dim=w.head_dim, full_workload_per_step=images == w.batch),
                cpu_baseline=dict(value=val, unit=UNIT, cores=torch.get_num_threads(), kind=kind, sample=sample),
                e2e=dict(value=val, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def run_reference_triton(args, w):
    """The reference's OWN Triton kernels on this GPU, untouched (no install()): fwd + bwd time on
    `w` and their error against the fp32 oracle on a small sample -- the bar to beat on the same
    box and the yardstick for this library's tolerances.  Returns a dict (with "unavailable" when
    the reference is not installed or its kernels do not compile for this GPU)."""
    if not os.path.isdir(os.path.join(REF_DIR, "flash_win_attn_v2")):
        return dict(impl="reference-triton", unavailable="the reference project is not installed under baseline/_ref")
    try:
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        import numpy as np
        from flash_win_attn_v2 import flash_win_attn_v2_func as ref_func
        from oracle import window_attention_oracle as orc
        dev = torch.device("cuda", 0)
        out = dict(impl="reference-triton", workload=w.name, dtype=w.dtype)

        def run(t):
            q, k, v = (t[x].detach().requires_grad_(True) for x in ("q", "k", "v"))
            ls, bias = t["logit_scale"].detach().requires_grad_(True), t["bias"].detach().requires_grad_(True)
            o = ref_func(q, k, v, ls, bias, t["mask"])
            return (o,) + torch.autograd.grad(o, (q, k, v, ls, bias), t["do"])

        # error against the fp32 oracle: two images of the workload's geometry
        small = Workload(w.name + "_sample", batch=2, nw=w.nw, heads=w.heads, window=w.window, dtype=w.dtype)
        ts = make_inputs(small, seed=0, device=dev)
        got = run(ts)
        f = lambda x: x.detach().float().cpu().numpy()
        ref = orc.forward_backward(*(f(ts[x]) for x in ("q", "k", "v", "do", "logit_scale", "bias", "mask")),
                                   dtype=np.float32)
        out["rel_err_vs_fp32_oracle"] = {name: float(orc.rel_err(f(g).reshape(ref[name].shape), ref[name]))
                                         for name, g in zip(("o", "dq", "dk", "dv", "dscale", "dbias"), got)}
        # time on the full workload
        t = make_inputs(w, seed=0, device=dev)
        for _ in range(3):
            run(t)
        torch.cuda.synchronize()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        evs = []
        for _ in range(max(3, min(args.steps, 10))):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run(t)
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in evs) / len(evs)
        out.update(ms_per_step=ms, tflops=w.matmul_flops() / (ms * 1e-3) / 1e12)
        return out
    except Exception as ex:
        return dict(impl="reference-triton", unavailable=f"{type(ex).__name__}: {str(ex)[:300]}")


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="cfg4", help="cfg2 | cfg3 | cfg4 | sweep_w<window>")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"],
                    help="reference: the classic path on the host cores; reference-triton: the reference's own "
                         "Triton kernels on this GPU (same-box yardstick, needs baseline/_ref)")
    ap.add_argument("--inputs", default="standard", choices=["standard", "reference_recipe"],
                    help="reference_recipe: the value distributions of the reference's own attention benchmark")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra configurations, the sweep and the model step")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = CONFIGS[args.config] if args.config in CONFIGS else sweep(int(args.config.split("_w")[1]))

    if args.impl == "reference":
        run_reference(args, w, rank)
        return
    if args.impl == "reference-triton":
        if rank == 0:
            print(json.dumps(run_reference_triton(args, w)), flush=True)
        return

    import torch.distributed as dist
    from flash_window_attention_v2_b200 import flash_win_attn_v2_func
    from flash_window_attention_v2_b200 import kernels as K
    from flash_window_attention_v2_b200.sharded import image_range, make_sharded_step

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    warmup = max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()

    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def flush_l2():
        flush_buf.zero_()

    def make_step(t):
        q, k, v = (t[x].detach().requires_grad_(True) for x in ("q", "k", "v"))
        ls = t["logit_scale"].detach().requires_grad_(True)
        bias = t["bias"].detach().requires_grad_(True)
        wrt = (q, k, v, ls, bias)

        def step():
            o = flash_win_attn_v2_func(q, k, v, ls, bias, t["mask"])
            return (o,) + torch.autograd.grad(o, wrt, t["do"])
        return step

    def time_steps(step, steps, warm):
        for _ in range(warm):
            step()
        torch.cuda.synchronize()
        barrier()
        evs = []
        for _ in range(steps):
            flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        barrier()
        ms = sum(a.elapsed_time(b) for a, b in evs)
        if world > 1:
            tt = torch.tensor([ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms / steps

    def kernel_times(t, steps, warm):
        """Device time of the forward kernel and of the backward main kernel alone (bare boundary
        calls, L2 flushed before every launch)."""
        q, k, v, do, ls = t["q"].detach(), t["k"].detach(), t["v"].detach(), t["do"], t["logit_scale"].detach()
        bias, mask = t["bias"].detach(), t["mask"]
        o, lse, _ = K._flash_attn_forward(q, k, v, ls, bias=bias, mask=mask, scale_type="tensor")
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        db, dscale = torch.empty_like(bias), torch.empty_like(ls)
        ws_bytes = K._lib.lib().fwa2_bwd_workspace_bytes(q.shape[0], q.shape[1], q.shape[2], mask.shape[0], 1, 1)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        bwd_full = lambda variant: K._flash_attn_backward(do, q, k, v, ls, o, lse, dq, dk, dv, dscale, db, bias=bias,
                                                          mask=mask, scale_type="tensor", _variant=variant,
                                                          _workspace=ws)
        bwd_full(0)
        fwd = lambda: K._flash_attn_forward(q, k, v, ls, bias=bias, mask=mask, scale_type="tensor")
        res = {}
        for name, fn in (("fwd", fwd), ("bwd_main", lambda: bwd_full(2 | 4)), ("bwd_all", lambda: bwd_full(0))):
            for _ in range(warm):
                fn()
            torch.cuda.synchronize()
            evs = []
            for _ in range(steps):
                flush_l2()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                evs.append((a, b))
            torch.cuda.synchronize()
            res[name] = sum(a.elapsed_time(b) for a, b in evs) / steps
        K.check_device_status(dev)
        return res

    def gen_inputs(wl, batch=None, seed=0):
        if args.inputs == "reference_recipe":
            assert batch is None or batch == wl.batch
            return make_reference_recipe_inputs(wl, seed=seed, device=dev)
        return make_inputs(wl, seed=seed, device=dev, batch=batch)

    # ------------------------------------------------------------------ the headline workload
    # One GPU: the whole workload.  N GPUs: rank r takes its contiguous share of the images.
    first_img, n_img = image_range(w.batch, world, rank) if world > 1 else (0, w.batch)
    t = gen_inputs(w, batch=n_img if world > 1 else None, seed=rank)
    sharded_parity = None
    if world == 1:
        step = make_step(t)
        api = "flash_win_attn_v2_func + torch.autograd.grad (eager)"
    else:
        step, sharded_parity, api = make_sharded_step(t, w, dev, K)
    with ClockSampler(local_rank) as clocks:
        ms_step = time_steps(step, args.steps, warmup)
        kt = kernel_times(t, max(5, args.steps // 3), 3) if rank == 0 else None
    K.check_device_status(dev)
    value = w.matmul_flops() / (ms_step * 1e-3) / 1e12      # the whole job: all ranks' windows / max-rank time

    # ------------------------------------------------------------------ end to end, host buffers
    # The same fwd + bwd through the package's host-buffer entry point: every step copies its
    # inputs from pinned host memory and its results (o, dq, dk, dv, dlogit_scale, dbias) back to
    # pinned host memory.  Consecutive steps overlap their copies and kernels on three streams;
    # the time is taken on the device from the first copy in to the last copy out.
    from flash_window_attention_v2_b200.host_io import HostBatchPipeline
    from flash_window_attention_v2_b200.sharded import sharded_flash_win_attn_v2_func
    host = {kk: (vv.detach().cpu().pin_memory() if vv is not None else None) for kk, vv in t.items()}
    pipe = HostBatchPipeline(dev, attn_func=(sharded_flash_win_attn_v2_func if world > 1 else flash_win_attn_v2_func))
    outs_host = None
    for _ in range(2):
        outs_host = pipe.submit(host)
    pipe.drain()
    # (as many steps as the device-timed loop: over a handful of steps the first copy in and the
    # last copy out, which overlap with nothing, are a fifth of the time)
    e2e_steps = max(3, min(args.steps, 30))
    torch.cuda.synchronize()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(pipe.s_in)
    for _ in range(e2e_steps):
        pipe.submit(host)
    ev1.record(pipe.s_out)
    pipe.drain()
    barrier()
    ms_e2e = ev0.elapsed_time(ev1)
    if world > 1:
        tt = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_e2e = float(tt.item())
    ms_e2e /= e2e_steps
    h2d = sum(v.numel() * v.element_size() for v in host.values() if v is not None)
    d2h = sum(b.numel() * b.element_size() for b in outs_host)
    e2e_val = w.matmul_flops() / (ms_e2e * 1e-3) / 1e12
    del pipe, host, outs_host

    # ------------------------------------------------------------------ the model step (config 5)
    model = None
    if not args.no_extra:
        try:
            model = model_step(dev, world, rank, K, barrier)
        except Exception as ex:      # an extra: never let it take the headline line down
            model = dict(error=f"{type(ex).__name__}: {ex}")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ------------------------------------------------------------------ roofline of the dominant kernel
    shard = Workload(w.name, batch=n_img, nw=w.nw, heads=w.heads, window=w.window, dtype=w.dtype)
    bwd_bytes = shard.algorithmic_bytes(fwd=False, bwd=True)
    ach = bwd_bytes / (kt["bwd_main"] * 1e-3) / 1e9
    traffic = NCU_TRAFFIC.get(w.name)
    roofline = dict(bound="hbm", kernel="bwd_quad_kernel" if 64 < w.n <= 256 else "bwd_kernel", achieved=ach,
                    peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"], peak_source=peaks["source"],
                    traffic=(traffic * n_img / w.batch) if traffic else None, launch_ms=kt["bwd_main"],
                    algorithmic_bytes_per_launch=bwd_bytes,
                    fwd_kernel=dict(launch_ms=kt["fwd"],
                                    achieved=shard.algorithmic_bytes(True, False) / (kt["fwd"] * 1e-3) / 1e9,
                                    frac=shard.algorithmic_bytes(True, False) / (kt["fwd"] * 1e-3) / 1e9 / peaks["hbm_gbs"]),
                    bwd_call_ms=kt["bwd_all"],
                    tensor_frac_of_bf16_peak=shard.matmul_flops() / ((kt["fwd"] + kt["bwd_all"]) * 1e-3) / 1e12
                    / peaks["bf16_tflops"])

    extra = {}
    if not args.no_extra and world == 1:
        from flash_window_attention_v2_b200.graphed import GraphedStep
        try:
            g = GraphedStep(t["q"], t["k"], t["v"], t["do"], t["logit_scale"], t["bias"], t["mask"])
            extra["graph_replay_ms_per_step"] = time_steps(g.replay, max(5, args.steps // 3), 3)
            del g
        except Exception as ex:
            extra["graph_replay_ms_per_step"] = f"{type(ex).__name__}: {ex}"
        del t
        torch.cuda.empty_cache()

        def point(wl, tx, steps=10):
            ms = time_steps(make_step(tx), steps, 3)
            ktx = kernel_times(tx, 5, 2)
            return dict(dtype=wl.dtype, n=wl.n, window_heads=wl.units, ms_per_step=ms,
                        tflops=wl.matmul_flops() / (ms * 1e-3) / 1e12,
                        frac_bf16_peak=wl.matmul_flops() / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                        hbm_frac_step=wl.algorithmic_bytes() / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                        fwd_kernel_ms=ktx["fwd"], bwd_kernel_ms=ktx["bwd_main"], bwd_call_ms=ktx["bwd_all"],
                        bwd_kernel_hbm_frac=wl.algorithmic_bytes(False, True) / (ktx["bwd_main"] * 1e-3) / 1e9
                        / peaks["hbm_gbs"],
                        binding="hbm" if wl.n <= 400 else "tensor / exp")

        for name in ("cfg2", "cfg3", "cfg4"):
            if name != w.name:
                wl = CONFIGS[name]
                extra[name] = point(wl, make_inputs(wl, seed=0, device=dev))
                torch.cuda.empty_cache()
        # the TFLOPS sweep of the reference's attention benchmark (batch 16 x 16 windows, 6 heads,
        # d 32; windows 8 .. 24), with this repository's inputs and with the reference's own recipe
        sw = {}
        for win in (8, 12, 16, 20, 24):
            wl = sweep(win)
            sw[f"w{win}"] = point(wl, make_inputs(wl, seed=0, device=dev), steps=8)
            wr = Workload(wl.name, batch=wl.batch, nw=wl.nw, heads=wl.heads, window=win, dtype="fp16")
            ms = time_steps(make_step(make_reference_recipe_inputs(wr, seed=0, device=dev)), 8, 3)
            sw[f"w{win}"]["reference_recipe_fp16"] = dict(
                ms_per_step=ms, tflops=wr.matmul_flops() / (ms * 1e-3) / 1e12,
                tflops_reference_convention=3 * (4 * wr.n * wr.n * 32 + 6 * wr.n * wr.n + 6 * wr.n * 32) * wr.units
                / (ms * 1e-3) / 1e12)
            torch.cuda.empty_cache()
        extra["sweep"] = sw
        K.check_device_status(dev)
    if model is not None:
        extra["swinv2_b_train_step"] = model
    if not args.no_extra and world == 1:
        # the reference's own Triton kernels on this box, in a process of their own
        for name in ("cfg3", "cfg4"):
            try:
                res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-triton",
                                      "--config", name, "--steps", "6"], capture_output=True, text=True, timeout=600)
                extra[f"reference_triton_{name}"] = json.loads(res.stdout.strip().splitlines()[-1])
            except Exception as ex:
                extra[f"reference_triton_{name}"] = dict(unavailable=f"{type(ex).__name__}: {str(ex)[:200]}")

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w)

    # forward (+ the pass that adds bias and mask into one fp32 table where the library uses one);
    # table transpose, backward, partial sums; (+ cross-GPU sum and cast)
    from flash_window_attention_v2_b200 import _lib
    combined = _lib.lib().fwa2_fwd_workspace_bytes(n_img * w.nw, w.heads, w.n, w.nw, 1, 1, 0) != 0
    launches = (4 if world == 1 else 5) + (1 if combined else 0)
    line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=warmup,
                ms_per_step=ms_step, higher_is_better=True, scaling="strong",
                vs_baseline=None, dtype=w.dtype, data="synthetic",
                config=dict(workload=w.name, inputs=args.inputs, images=w.batch, images_on_rank0=n_img,
                            windows_per_image=w.nw, heads=w.heads, n=w.n, head_dim=w.head_dim,
                            window_heads=w.units, sharding=None if world == 1 else "images split over ranks",
                            l2="256 MiB buffer rewritten before every timed step", api=api),
                frac_bf16_peak=value / world / peaks["bf16_tflops"],
                hbm_frac_step=w.algorithmic_bytes() / world / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                roofline=roofline, cpu_baseline=cpu,
                e2e=dict(value=e2e_val, unit=UNIT, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, ms_per_step=ms_e2e),
                gpu_launches=launches * args.steps, gpu_launches_per_step=launches,
                sharded_parity=sharded_parity, clocks=clocks.summary(), extra=extra)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def model_step(dev, world, rank, K, barrier, batch_per_gpu: int = 16, steps: int = 4):
    """SwinV2-B training step (patch 4, embed 128, depths 2-2-18-2, heads 4-8-16-32, window 16, bf16,
    random init, 256 x 256 inputs) with the REFERENCE's own model code, every WindowAttention call
    routed through these kernels by install(); plain DDP over the ranks.  Images per second, and the
    same step on the reference's classic path (`is_flash=False`) beside it.  Needs the reference
    installed under baseline/_ref."""
    if not os.path.isdir(os.path.join(REF_DIR, "flash_win_attn_v2")):
        return dict(unavailable="the reference project is not installed under baseline/_ref")
    import torch.nn.functional as F
    from flash_window_attention_v2_b200 import install
    install()
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    from flash_win_attn_v2 import SwinTransformerV2
    cfg = dict(img_size=256, patch_size=4, embed_dim=128, depths=[2, 2, 18, 2], num_heads=[4, 8, 16, 32],
               window_size=16)
    out = dict(model="SwinV2-B", batch_per_gpu=batch_per_gpu, n_gpus=world, dtype="bf16", **{k: str(v) for k, v in cfg.items()})
    for name, flash in (("these_kernels", True), ("classic_path_on_gpu", False)):
        torch.manual_seed(0)
        m = SwinTransformerV2(**cfg, is_flash=flash).to(device=dev, dtype=torch.bfloat16)
        if world > 1:
            m = torch.nn.parallel.DistributedDataParallel(m, device_ids=[dev.index])
        opt = torch.optim.Adam(m.parameters(), lr=1e-4)
        x = torch.randn(batch_per_gpu, 3, 256, 256, device=dev, dtype=torch.bfloat16)
        y = torch.randint(0, 1000, (batch_per_gpu,), device=dev)

        def train():
            opt.zero_grad()
            loss = F.cross_entropy(m(x), y)
            loss.backward()
            opt.step()
            return loss
        for _ in range(2):
            train()
        torch.cuda.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            loss = train()
        b.record()
        torch.cuda.synchronize()
        barrier()
        ms = a.elapsed_time(b) / steps
        if world > 1:
            import torch.distributed as dist
            tt = torch.tensor([ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        out[name] = dict(ms_per_step=ms, images_per_s=batch_per_gpu * world / (ms * 1e-3), loss=float(loss))
        del m, opt
        torch.cuda.empty_cache()
    K.check_device_status(dev)
    out["speedup_vs_classic"] = out["classic_path_on_gpu"]["ms_per_step"] / out["these_kernels"]["ms_per_step"]
    return out


if __name__ == "__main__":
    main()
