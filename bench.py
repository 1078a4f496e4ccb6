#!/usr/bin/env python
"""Benchmark of the window-attention hot path: forward + backward TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config cfg2] [--impl ours|reference]

One "step" is one forward + backward pass of the op over one batch of synthetic windows, through
the public autograd API.  With N > 1 (launched by torch.distributed.run, one rank per GPU) every
rank works on its own full-size batch (weak scaling); the only exchange step is the all-reduce of
dBias / dLogitScale inside backward.  Rank 0 prints ONE JSON line.

`--impl reference` times the reference's classic PyTorch path on the host CPU cores (the
multi-threaded port in oracle/classic_cpu.py) on a bounded sample of the same workload.
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

from flash_window_attention_v2_b200.workloads import CONFIGS, make_inputs, sweep  # noqa: E402

METRIC = "fwd+bwd window-attention throughput (matmul FLOPs 14*N^2*d per window-head)"
UNIT = "TFLOP/s"


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


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core it may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))


def cpu_baseline(w, seconds: float = 12.0, sample_images: int | None = None):
    """Times oracle/classic_cpu.py (fp32, all host threads) on `sample_images` images of `w`."""
    use_all_host_threads()
    from oracle import classic_cpu
    if sample_images is None:
        # aim at roughly a second per pass: the classic path materialises (BW, H, N, N) fp32
        per_image = w.nw * w.heads * w.n * w.n * 4
        sample_images = max(1, min(w.batch, int(1.5e8 // per_image)))
    t = make_inputs(w, seed=0, batch=sample_images)
    f = {k: (v.float() if v is not None else None) for k, v in t.items()}
    flops = 14.0 * w.n * w.n * w.head_dim * sample_images * w.nw * w.heads
    classic_cpu.forward_backward(f["q"], f["k"], f["v"], f["do"], f["logit_scale"], f["bias"], f["mask"])
    n, t0 = 0, time.perf_counter()
    while True:
        classic_cpu.forward_backward(f["q"], f["k"], f["v"], f["do"], f["logit_scale"], f["bias"], f["mask"])
        n += 1
        el = time.perf_counter() - t0
        if el >= seconds or n >= 200:
            break
    return dict(value=flops * n / el / 1e12, unit=UNIT, cores=torch.get_num_threads(), kind="port",
                sample=f"{sample_images} of {w.batch} images ({sample_images * w.nw * w.heads} window-heads), "
                       f"{n} passes in {el:.1f} s, fp32, host cpu_count={os.cpu_count()}",
                seconds_per_full_step=el / n * w.batch / sample_images)


def run_reference(args, w, rank):
    """The reference arm: its classic path on the host cores; rank 0 only."""
    if rank != 0:
        return
    use_all_host_threads()
    per_image = w.nw * w.heads * w.n * w.n * 4
    sample_images = max(1, min(w.batch, int(1.5e8 // per_image)))
    from oracle import classic_cpu
    t = make_inputs(w, seed=0, batch=sample_images)
    f = {k: (v.float() if v is not None else None) for k, v in t.items()}
    flops = 14.0 * w.n * w.n * w.head_dim * sample_images * w.nw * w.heads
    for _ in range(max(1, min(args.warmup, 3))):
        classic_cpu.forward_backward(f["q"], f["k"], f["v"], f["do"], f["logit_scale"], f["bias"], f["mask"])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        classic_cpu.forward_backward(f["q"], f["k"], f["v"], f["do"], f["logit_scale"], f["bias"], f["mask"])
    el = time.perf_counter() - t0
    val = flops * args.steps / el / 1e12
    sample = (f"each step = {sample_images} of {w.batch} images ({sample_images * w.nw * w.heads} window-heads) "
              f"of {w.name}, fp32 classic path on host cores")
    line = dict(impl="reference", metric=METRIC, value=val, unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=el / args.steps * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=w.name, window_heads_per_step=sample_images * w.nw * w.heads, n=w.n,
                            head_dim=w.head_dim),
                cpu_baseline=dict(value=val, unit=UNIT, cores=torch.get_num_threads(), kind="port", sample=sample),
                e2e=dict(value=val, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="cfg2", help="cfg2 | cfg3 | cfg4 | sweep_w<window>")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra single-GPU configurations")
    ap.add_argument("--no-graph", action="store_true", help="time the eager step instead of the CUDA-graph replay")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = CONFIGS[args.config] if args.config in CONFIGS else sweep(int(args.config.split("_w")[1]))

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    import torch.distributed as dist
    from flash_window_attention_v2_b200 import flash_win_attn_v2_func
    from flash_window_attention_v2_b200 import kernels as K
    from flash_window_attention_v2_b200.sharded import sharded_flash_win_attn_v2_func

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()

    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def flush_l2():
        flush_buf.zero_()

    def make_step(wl, t):
        q, k, v = (t[x].requires_grad_(True) for x in ("q", "k", "v"))
        ls = t["logit_scale"].requires_grad_(True)
        bias = t["bias"].requires_grad_(True)
        wrt = (q, k, v, ls, bias)

        def step():
            if world > 1:
                o = sharded_flash_win_attn_v2_func(q, k, v, ls, bias, t["mask"])
            else:
                o = flash_win_attn_v2_func(q, k, v, ls, bias, t["mask"])
            return (o,) + torch.autograd.grad(o, wrt, t["do"])
        return step

    def time_steps(step, steps, warmup):
        for _ in range(warmup):
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

    def kernel_times(wl, t, steps, warmup):
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
            for _ in range(warmup):
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

    # ------------------------------------------------------------------ the headline workload
    t = make_inputs(w, seed=rank, device=dev)
    step = make_step(w, t)
    # One GPU: the step (flash_win_attn_v2_func + torch.autograd.grad, four kernels) is captured once
    # into a CUDA graph and replayed, so that the host's trip through autograd and ctypes is not
    # what gets timed; the eager number is reported next to it.  More than one GPU: the same local
    # kernels in a graph, followed (outside the graph) by the NCCL all-reduce of the parameter
    # gradients and the cast kernel.
    api = "flash_win_attn_v2_func + torch.autograd.grad"
    ms_eager = None
    graphed = None
    if not args.no_graph:
        try:
            if world == 1:
                from flash_window_attention_v2_b200.graphed import GraphedStep
                graphed = GraphedStep(t["q"], t["k"], t["v"], t["do"], t["logit_scale"], t["bias"], t["mask"])
            else:
                # the local kernels in a graph; the all-reduce of the parameter gradients and the
                # cast that follows it stay outside (nothing that waits for a peer is captured)
                from flash_window_attention_v2_b200.sharded import GraphedShardedStep
                graphed = GraphedShardedStep(t["q"], t["k"], t["v"], t["do"], t["logit_scale"], t["bias"], t["mask"])
        except Exception as ex:   # capture refused: say so and time the eager step
            print(f"bench: CUDA graph capture failed ({type(ex).__name__}: {ex}); timing the eager step", file=sys.stderr)
            graphed = None
    with ClockSampler(local_rank) as clocks:
        if graphed is not None:
            ms_eager = time_steps(step, max(5, args.steps // 2), 3)
            ms_step = time_steps(graphed.replay, args.steps, max(args.warmup, 3))
            api = ("flash_win_attn_v2_func + torch.autograd.grad, captured in a CUDA graph (GraphedStep) and replayed"
                   if world == 1 else
                   "GraphedShardedStep: local kernels replayed from a CUDA graph, then NCCL all-reduce + cast")
        else:
            ms_step = time_steps(step, args.steps, max(args.warmup, 3))
        kt = kernel_times(w, t, max(5, args.steps // 2), 3) if rank == 0 or world == 1 else None
    K.check_device_status(dev)
    flops_rank = w.matmul_flops()
    value = flops_rank * world / (ms_step * 1e-3) / 1e12

    # ------------------------------------------------------------------ end to end, host buffers
    # The same fwd + bwd through the package's host-buffer entry point: every step copies its
    # inputs from pinned host memory and its results (o, dq, dk, dv, dlogit_scale, dbias) back to
    # pinned host memory.  Consecutive steps overlap their copies and kernels on three streams;
    # the time is taken on the device from the first copy in to the last copy out.  The inputs
    # (about 200 MB per step) come over PCIe every step, so no step can find them in L2.
    from flash_window_attention_v2_b200.host_io import HostBatchPipeline
    host = {kk: (vv.detach().cpu().pin_memory() if vv is not None else None) for kk, vv in t.items()}
    pipe = HostBatchPipeline(dev, attn_func=(sharded_flash_win_attn_v2_func if world > 1 else flash_win_attn_v2_func))
    outs_host = None
    for _ in range(3):
        outs_host = pipe.submit(host)
    pipe.drain()
    e2e_steps = max(4, min(args.steps, 12))
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
    e2e_val = flops_rank * world / (ms_e2e * 1e-3) / 1e12

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ------------------------------------------------------------------ roofline of the dominant kernel
    # DRAM bytes per launch of the dominant kernel from the ncu captures summarised in profiles/
    # (dram__bytes_read.sum + dram__bytes_write.sum); None for workloads that were not captured
    ncu_traffic = {"cfg2": 368.9e6, "cfg3": 198.7e6}
    bwd_bytes = w.algorithmic_bytes(fwd=False, bwd=True)
    ach = bwd_bytes / (kt["bwd_main"] * 1e-3) / 1e9
    roofline = dict(bound="hbm", kernel="bwd_kernel", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s",
                    frac=ach / peaks["hbm_gbs"], peak_source=peaks["source"], traffic=ncu_traffic.get(w.name),
                    launch_ms=kt["bwd_main"], algorithmic_bytes_per_launch=bwd_bytes,
                    fwd_kernel=dict(launch_ms=kt["fwd"],
                                    achieved=w.algorithmic_bytes(True, False) / (kt["fwd"] * 1e-3) / 1e9,
                                    frac=w.algorithmic_bytes(True, False) / (kt["fwd"] * 1e-3) / 1e9 / peaks["hbm_gbs"]),
                    bwd_call_ms=kt["bwd_all"],
                    tensor_frac_of_bf16_peak=w.matmul_flops() / ((kt["fwd"] + kt["bwd_all"]) * 1e-3) / 1e12
                    / peaks["bf16_tflops"])

    extra = {}
    if not args.no_extra and world == 1:
        for name in ("cfg3", "cfg4", "cfg2"):
            if name == w.name:
                continue
            wl = CONFIGS[name]
            tx = make_inputs(wl, seed=0, device=dev)
            ms = time_steps(make_step(wl, tx), 10, 3)
            ktx = kernel_times(wl, tx, 5, 2)
            extra[name] = dict(dtype=wl.dtype, n=wl.n, window_heads=wl.units, ms_per_step=ms,
                               tflops=wl.matmul_flops() / (ms * 1e-3) / 1e12,
                               frac_bf16_peak=wl.matmul_flops() / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                               fwd_kernel_ms=ktx["fwd"], bwd_kernel_ms=ktx["bwd_main"], bwd_call_ms=ktx["bwd_all"],
                               kernels_tflops=wl.matmul_flops() / ((ktx["fwd"] + ktx["bwd_all"]) * 1e-3) / 1e12,
                               kernels_hbm_frac=wl.algorithmic_bytes() / ((ktx["fwd"] + ktx["bwd_all"]) * 1e-3) / 1e9
                               / peaks["hbm_gbs"])
            del tx
            torch.cuda.empty_cache()

    # the bias-preparation step in front of the operator (not part of the headline metric): fused
    # kernels against the reference's own torch expression, both on this GPU
    if not args.no_extra and world == 1:
        try:
            from flash_window_attention_v2_b200.cpb_bias import cpb_bias_backward, cpb_bias_forward
            from oracle.window_attention_oracle import relative_position_index
            side = int(round(math.sqrt(w.n)))
            if side * side == w.n:
                idx = torch.from_numpy(relative_position_index(side, side)).to(dev)
                tab = torch.randn((2 * side - 1) ** 2, w.heads, device=dev).to(t["q"].dtype)
                dbf = torch.randn(w.heads, w.n, w.n, device=dev)

                def torch_expr():
                    tt = tab.detach().requires_grad_(True)
                    b = 16 * torch.sigmoid(tt[idx.view(-1)].view(w.n, w.n, -1).permute(2, 0, 1).contiguous())
                    return torch.autograd.grad(b, tt, dbf.to(b.dtype))

                def fused():
                    cpb_bias_forward(tab, idx, tab.dtype)
                    return cpb_bias_backward(dbf, tab, idx, tab.dtype)

                extra["cpb_bias_step"] = dict(n=w.n, heads=w.heads, fused_fwd_bwd_ms=time_steps(fused, 10, 3),
                                              torch_expression_fwd_bwd_ms=time_steps(torch_expr, 10, 3))
        except Exception as ex:   # an extra: never let it take the headline line down
            extra["cpb_bias_step"] = dict(error=f"{type(ex).__name__}: {ex}")

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w)

    line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype=w.dtype,
                data="synthetic",
                config=dict(workload=w.name, images_per_gpu=w.batch, windows_per_image=w.nw, heads=w.heads, n=w.n,
                            head_dim=w.head_dim, window_heads_per_gpu=w.units,
                            l2="256 MiB buffer rewritten before every timed step",
                            api=api, eager_ms_per_step=ms_eager),
                frac_bf16_peak=value / world / peaks["bf16_tflops"],
                hbm_frac_step=w.algorithmic_bytes() / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                roofline=roofline, cpu_baseline=cpu,
                e2e=dict(value=e2e_val, unit=UNIT, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, ms_per_step=ms_e2e),
                gpu_launches=((5 if world > 1 else 4) * args.steps),   # inside the timed region of `value`
                gpu_launches_per_step=(5 if world > 1 else 4), clocks=clocks.summary(), extra=extra)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
