#!/usr/bin/env python
"""Benchmark: causal attention forward + backward, bf16, B=64 H=16 T=4096 D=128, heads sharded over GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  A "step" is one forward + backward pass over this rank's shard of
the batch*head axis.  `value` is causal-adjusted TFLOP/s of the whole job (forward 2*BH*T^2*D,
backward 5*BH*T^2*D) with operands resident in HBM; `e2e` is the same metric through the host-buffer
pipeline (pinned host memory in, host memory out, copies inside the timed region).
For N > 1 launch with torchrun (one rank per GPU); a bare `python bench.py --gpus N` re-launches itself.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "causal attention fwd+bwd TFLOP/s (bf16, T=4096, d=128; causal-adjusted 7*B*H*T^2*D flops)"
UNIT = "TFLOP/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c5", help="workload from inferno_b200.synth.CONFIGS (bf16 ones)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=64, help="heads per chunk of the host pipeline")
    ap.add_argument("--e2e-nbuf", type=int, default=2, help="device staging sets of the host pipeline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def peaks():
    """Measured roofline denominators (driver-written file), else the documented fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16_sustained=float(p["bf16_tflops_sustained"]), bf16_burst=float(p["bf16_tflops"]),
                    hbm_gbs=float(p["hbm_gbs"]), source="measured")
    return dict(bf16_sustained=1400.0, bf16_burst=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """SM clock under load and throttle reasons, read (never set) through NVML every 2 ms on a thread while the timed
    region runs; falls back to polling nvidia-smi when the NVML binding is missing."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples, self.power, self.mask = [], [], 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._smi = None
        self.lines = []

    def _nvml_loop(self, nv, handle):
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                self.power.append(nv.nvmlDeviceGetPowerUsage(handle) / 1000.0)
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(handle))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.gpu]) if visible and visible.split(",")[self.gpu].isdigit() else self.gpu
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        try:
            fields = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                      "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                      "clocks_event_reasons.sw_power_cap")
            self._smi = subprocess.Popen(["nvidia-smi", f"--query-gpu={fields}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: [self.lines.append(x.strip()) for x in self._smi.stdout], daemon=True).start()
        except OSError:
            self._smi = None

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            reasons = sorted(name for name, bit in self.REASONS if self.mask & bit)
            return dict(sm_mhz=statistics.median(self.samples) if self.samples else None, sm_max_mhz=self.max_mhz,
                        power_w_max=max(self.power) if self.power else None, samples=len(self.samples), reasons=reasons,
                        source="nvml")
        if self._smi is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no clock source available"], samples=0)
        self._smi.terminate()
        try:
            self._smi.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._smi.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    power_w_max=max(power) if power else None, samples=len(sm), reasons=sorted(reasons), source="nvidia-smi")


# ----------------------------------------------------------------------------------------------
# CPU legs (the reference's own CPU path when oracle/_ref is built, else the C restatement)
# ----------------------------------------------------------------------------------------------
def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample(cfg, T_sample: int, procs: int, seed: int = 0):
    """Run `procs` heads of shape [T_sample, D] through the CPU implementation, one head per
    process/thread, and return (causal-adjusted TFLOP/s, kind, seconds)."""
    import numpy as np
    from oracle import oracle as orc
    from inferno_b200.synth import make_inputs
    D = cfg.D
    flops = 7.0 * procs * float(T_sample) ** 2 * D
    if orc.have_ref():
        with tempfile.TemporaryDirectory() as td:
            q, k, v, do = make_inputs(1, 1, T_sample, D, cfg.seed + seed, cfg.qkv_std, cfg.do_std, cfg.dtype)
            for name, arr in (("q", q), ("k", k), ("v", v), ("do", do)):
                arr.tofile(os.path.join(td, name + ".bin"))
            t0 = time.perf_counter()
            ps = [subprocess.Popen([orc.REF_BIN, "cpu", "1", "1", str(T_sample), str(D), os.path.join(td, "q.bin"),
                                    os.path.join(td, "k.bin"), os.path.join(td, "v.bin"), os.path.join(td, "do.bin"),
                                    os.path.join(td, f"out{i}")], stdout=subprocess.DEVNULL, cwd=td) for i in range(procs)]
            rcs = [p.wait() for p in ps]
            dt = time.perf_counter() - t0
        if any(rcs):
            raise RuntimeError("oracle/_ref/ref_attention failed")
        return flops / dt / 1e12, "reference", dt
    q, k, v, do = make_inputs(procs, 1, T_sample, D, cfg.seed + seed, cfg.qkv_std, cfg.do_std, cfg.dtype)
    t0 = time.perf_counter()
    orc.oracle_f32(q, k, v, do, scale=cfg.scale, threads=procs)
    dt = time.perf_counter() - t0
    return flops / dt / 1e12, "port", dt


def pick_sample_T(cfg, budget_s: float) -> int:
    """Largest prefix length whose one-head-per-core pass is expected to fit the budget
    (the reference CPU path measured ~8 s per head at T=2048, D=128, growing with T^2)."""
    T = cfg.T
    while T > 256 and 8.5 * (T / 2048.0) ** 2 * (cfg.D / 128.0) > budget_s:
        T //= 2
    return T


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = min(host_cores(), 64)
    budget = max(2.0, 150.0 / max(1, args.steps + args.warmup))
    T_s = pick_sample_T(cfg, budget)
    kind = "port"
    for i in range(args.warmup):
        _, kind, _ = cpu_sample(cfg, T_s, cores, seed=i)
    vals, secs = [], []
    for i in range(args.steps):
        v, kind, dt = cpu_sample(cfg, T_s, cores, seed=100 + i)
        vals.append(v); secs.append(dt)
    total_flops = 7.0 * cores * float(T_s) ** 2 * cfg.D * args.steps
    value = total_flops / sum(secs) / 1e12 if secs else 0.0
    sample = (f"{cores} heads per step, one per host core, each the first {T_s} positions of a "
              f"T={cfg.T} D={cfg.D} causal head (a causal prefix is a self-contained sub-problem)")
    line = dict(impl="reference", metric=METRIC, value=value, unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * sum(secs) / max(1, len(secs)), higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                config=workload_config(cfg, args.gpus),
                cpu_baseline=dict(value=value, unit=UNIT, cores=cores, kind=kind, sample=sample),
                e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def workload_config(cfg, n_gpus):
    return dict(workload=f"{cfg.name}: causal self-attention fwd+bwd, bf16 I/O fp32 accumulate, B={cfg.B} H={cfg.H} "
                         f"T={cfg.T} d_head={cfg.D}, batch*head axis partitioned over {n_gpus} GPU(s)",
                B=cfg.B, H=cfg.H, T=cfg.T, D=cfg.D, parallelism=f"heads/{n_gpus}", collective_in_path="none",
                l2="operands (>=128 MiB per tensor per rank) exceed the 126 MB L2; no flush needed")


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def run_ours(args, cfg):
    import torch
    import torch.distributed as dist
    from inferno_b200 import attention as A
    from inferno_b200.host_pipeline import HostAttention
    from inferno_b200.shard import shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    BH = cfg.B * cfg.H
    heads = shard_range(BH, rank, world)
    n, T, D = len(heads), cfg.T, cfg.D
    g = torch.Generator(device=dev).manual_seed(cfg.seed * 1000 + rank)
    mk = lambda std: (torch.randn(n, 1, T, D, device=dev, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
    q, k, v, do = mk(cfg.qkv_std), mk(cfg.qkv_std), mk(cfg.qkv_std), mk(cfg.do_std)
    o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty(n, 1, T, device=dev, dtype=torch.float32)

    def step():
        A.attention_forward(q, k, v, out=o, lse=lse)
        A.attention_backward(q, k, v, o, do, lse, dq=dq, dk=dk, dv=dv)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    A.check_device_status()

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K)]
    for row in ev:      # create the underlying CUDA events outside the timed region
        for e in row:
            e.record()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    t0.record()
    for i in range(K):
        A.set_timing_events(*ev[i])
        step()
    t1.record()
    barrier()
    clocks = sampler.stop()
    A.set_timing_events()
    A.check_device_status()
    ms_total = t0.elapsed_time(t1)
    fwd_ms = statistics.mean(ev[i][0].elapsed_time(ev[i][1]) for i in range(K))
    bwd_ms = statistics.mean(ev[i][2].elapsed_time(ev[i][3]) for i in range(K))
    t = torch.tensor([ms_total / K, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, fwd_ms_max, bwd_ms_max = (float(x) for x in t.tolist())
    total_flops = cfg.flops()
    value = total_flops / (ms_step * 1e-3) / 1e12

    # ---- end to end: pinned host buffers in, host buffers out, copies inside the timed region ----
    if args.e2e_steps <= 0:      # profiling runs only; a bench line without e2e is not a result
        e2e = None
    else:
        e2e = measure_e2e(args, torch, dist, A, HostAttention, dev, world, n, T, D, (q, k, v, do), o, barrier, total_flops)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    finish(args, cfg, world, n, T, D, K, value, ms_step, fwd_ms_max, bwd_ms_max, clocks, e2e, total_flops, dist)


def measure_e2e(args, torch, dist, A, HostAttention, dev, world, n, T, D, operands, o, barrier, total_flops):
    q, k, v, do = operands
    hc = max(1, min(n, args.e2e_heads_per_chunk))
    pipe = HostAttention(hc, T, D, torch.bfloat16, dev, nbuf=args.e2e_nbuf)
    hin = [torch.empty((n, 1, T, D), dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    hout = [torch.empty((n, 1, T, D), dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    for h_, d_ in zip(hin, (q, k, v, do)):
        h_.copy_(d_)
    pipe.run(*hin, *hout)                      # warm-up (also first touch of the pinned pages)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    Ke = max(1, args.e2e_steps)
    e0.record()
    for _ in range(Ke):
        pipe.run(*hin, *hout)
    e1.record()
    barrier()
    te = torch.tensor([e0.elapsed_time(e1) / Ke], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item())
    shard_bytes = n * T * D * 2
    e2e_check = float((hout[0][:1].float() - o[:1].float().cpu()).abs().max())   # pipeline output == resident output
    return dict(value=total_flops / (e2e_ms * 1e-3) / 1e12, unit=UNIT, ms_per_step=e2e_ms, steps=Ke,
                h2d_bytes_per_step=4 * shard_bytes, d2h_bytes_per_step=4 * shard_bytes,
                api="inferno_b200.host_pipeline.HostAttention.run (pinned host in/out, 3-stream chunked pipeline over the C ABI)",
                max_abs_diff_vs_resident=e2e_check)


def finish(args, cfg, world, n, T, D, K, value, ms_step, fwd_ms_max, bwd_ms_max, clocks, e2e, total_flops, dist):
    pk = peaks()
    bwd_flops_rank = 5.0 * n * float(T) ** 2 * D
    achieved = bwd_flops_rank / (bwd_ms_max * 1e-3) / 1e12
    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=K, warmup=max(args.warmup, 3), ms_per_step=ms_step,
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
        config=workload_config(cfg, world),
        per_gpu_tflops=value / world,
        fwd=dict(ms=fwd_ms_max, tflops=2.0 * n * float(T) ** 2 * D / (fwd_ms_max * 1e-3) / 1e12),
        bwd_main=dict(ms=bwd_ms_max, tflops=achieved),
        frac_of_bf16_peak=dict(value=value / world / pk["bf16_sustained"], peak_tflops=pk["bf16_sustained"],
                               of=pk["source"] + " sustained cuBLAS bf16", nominal_frac=value / world / 2250.0),
        clocks=clocks,
        e2e=e2e,
        gpu_launches=4 * K,
        kernels_per_step=["attn_fwd_persist_kernel", "delta_kernel", "attn_bwd_persist_kernel", "dq_finish_kernel"],
        roofline=dict(bound="tensor", kernel=f"attn_bwd_persist_kernel<D={D}>", achieved=achieved, peak=pk["bf16_sustained"],
                      unit="TFLOP/s", frac=achieved / pk["bf16_sustained"], of=pk["source"],
                      algorithmic_flops_per_launch=bwd_flops_rank, traffic=TRAFFIC_BYTES_PER_ELEMENT * n * T * D if TRAFFIC_BYTES_PER_ELEMENT else None,
                      traffic_source="ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on c3 "
                                     "(profiles/attn_bwd_persist_kernel_c3_bf16_T8192_D128.md), scaled by elements per launch"),
    )
    if world == 1 and not args.no_cpu_baseline:
        try:
            cores = min(host_cores(), 64)
            T_s = pick_sample_T(cfg, 45.0)
            val, kind, dt = cpu_sample(cfg, T_s, cores)
            line["cpu_baseline"] = dict(value=val, unit=UNIT, cores=cores, kind=kind, seconds=dt,
                                        sample=f"{cores} heads, one per host core, each the first {T_s} positions of a T={cfg.T} "
                                               f"D={cfg.D} causal head, fp32 (the reference has no bf16)")
        except Exception as exc:   # the CPU leg must never take the GPU numbers down with it
            line["cpu_baseline"] = dict(value=None, unit=UNIT, cores=0, kind="port", sample=f"failed: {exc}")
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + write) of one attn_bwd_persist_kernel launch per element of a [heads, T, D] operand, from the
# ncu capture summarised in profiles/attn_bwd_persist_kernel_c3_bf16_T8192_D128.md: (408.2 + 230.3) MB over
# 32 heads x 8192 x 128 elements.  DRAM traffic of this kernel is proportional to the elements it touches
# (each operand is read once from DRAM; re-reads by other CTAs of a head hit L2).
TRAFFIC_BYTES_PER_ELEMENT = (408.220928e6 + 230.287872e6) / (32 * 8192 * 128)


def main():
    args = parse_args()
    from inferno_b200.synth import CONFIGS
    cfg = CONFIGS[args.config]
    if cfg.dtype != "bf16":
        raise SystemExit("bench configs are the bf16 ones (c5, c3, c4_layer)")
    if args.impl == "reference":
        run_reference(args, cfg)
        return
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    run_ours(args, cfg)


if __name__ == "__main__":
    main()
