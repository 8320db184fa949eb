#!/usr/bin/env python
"""Benchmark: causal attention forward + backward, heads sharded over the GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c5|c3|c4_layer|c2]

Prints ONE JSON line (rank 0).  A "step" is one forward + backward pass over this rank's shard of the batch*head
axis.  `value` is causal-adjusted TFLOP/s of the whole job (forward 2*BH*T^2*D, backward 5*BH*T^2*D) with operands
resident in HBM; `e2e` is the same metric through the host-buffer pipeline (pinned host memory in, host memory out,
copies inside the timed region).  Default workload: c5 = bf16, B=64 H=16 T=4096 D=128.

What a run does, in order: generate every head's operands on the host from the head's own seeded stream (identical
at every N), copy them in, W warm-up steps, further untimed steps until the GPU has been under load for
--min-load-seconds (so that every N is timed in the same, settled power state), EXACTLY K timed steps between two
CUDA events, the end-to-end pipeline and its copy-only floor, and -- outside every timed region -- the validation:
each rank checks the first and last head of its shard against a float64 evaluation, 64-bit checksums of O, dK and dV
of every head are gathered over NCCL, and their digest is printed (it must not depend on N).
For N > 1 launch with torchrun (one rank per GPU); a bare `python bench.py --gpus N` re-launches itself.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

UNIT = "TFLOP/s"
# Every CPU leg (the reference arm and the cpu_baseline object of the GPU arm) times heads cut to this many positions
# when the configuration's T is longer: a causal prefix is a self-contained sub-problem, and a full T = 4096 head takes
# the reference's CPU path about 35 s.
CPU_SAMPLE_T = 1024
L2_BYTES = 126 * 1000 * 1000


def metric_name(cfg) -> str:
    io = "bf16" if cfg.dtype == "bf16" else "fp32 I/O, split-bf16 products"
    return f"causal attention fwd+bwd TFLOP/s ({io}, T={cfg.T}, d={cfg.D}; causal-adjusted 7*B*H*T^2*D flops)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c5", help="workload from inferno_b200.synth.CONFIGS")
    ap.add_argument("--min-load-seconds", type=float, default=2.0,
                    help="untimed steps run before the timed ones until the GPU has been busy this long")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=0, help="heads per chunk of the host pipeline (0: shard / 8)")
    ap.add_argument("--e2e-nbuf", type=int, default=3, help="device staging sets of the host pipeline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-validate", action="store_true")
    ap.add_argument("--no-cuda-graph", action="store_true", help="skip the CUDA-graph replay measured for small configurations")
    ap.add_argument("--ref-cuda", action="store_true", help="also time the reference's own CUDA path (small fp32 configs only)")
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


def workload_config(cfg, n_gpus):
    T_cpu = min(cfg.T, CPU_SAMPLE_T)
    io = "bf16 I/O fp32 accumulate" if cfg.dtype == "bf16" else "fp32 I/O, products as three bf16 MMAs (hi/lo split), fp32 accumulate"
    cpu = (f"CPU legs time whole heads (T={cfg.T})" if T_cpu == cfg.T else
           f"CPU legs time the first {T_cpu} positions of a head (a causal prefix is a self-contained sub-problem)")
    heads_bytes = cfg.B * cfg.H // max(1, n_gpus) * cfg.T * cfg.D * (2 if cfg.dtype == "bf16" else 4)
    l2 = ("operands of one tensor per rank exceed the 126 MB L2; no flush needed" if heads_bytes > L2_BYTES else
          "a 256 MB buffer is written between timed steps (operands would fit in the 126 MB L2); steps are timed one by one")
    return dict(workload=f"{cfg.name}: causal self-attention fwd+bwd, {io}, B={cfg.B} H={cfg.H} T={cfg.T} d_head={cfg.D}, "
                         f"batch*head axis partitioned over {n_gpus} GPU(s); every head's Q, K, V, dO from its own stream "
                         f"numpy default_rng([{cfg.seed}, head]); {cpu}",
                B=cfg.B, H=cfg.H, T=cfg.T, D=cfg.D, parallelism=f"heads/{n_gpus}", collective_in_path="none", l2=l2,
                cpu_sample_T=T_cpu)


# ----------------------------------------------------------------------------------------------
# CPU legs (the reference's own CPU path when oracle/_ref is built, else the C restatement)
# ----------------------------------------------------------------------------------------------
def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _cpu_head_inputs(cfg, head, T_sample):
    from inferno_b200.synth import make_head_inputs
    return tuple(a[:T_sample] for a in make_head_inputs(cfg, head))


def _cpu_heads(cfg, first_head, count, T_sample):
    total = cfg.B * cfg.H
    with ThreadPoolExecutor(min(16, host_cores())) as ex:
        return list(ex.map(lambda i: _cpu_head_inputs(cfg, (first_head + i) % total, T_sample), range(count)))


def cpu_sample(cfg, T_sample: int, procs: int, first_head: int = 0):
    """Run `procs` heads of shape [T_sample, D] through the CPU implementation, one head per process (reference) or
    thread (port), and return (causal-adjusted TFLOP/s, kind, seconds)."""
    import numpy as np
    from oracle import oracle as orc
    D = cfg.D
    flops = 7.0 * procs * float(T_sample) ** 2 * D
    if orc.have_ref():
        with tempfile.TemporaryDirectory() as td:
            for i, parts in enumerate(_cpu_heads(cfg, first_head, procs, T_sample)):
                for name, arr in zip(("q", "k", "v", "do"), parts):
                    np.ascontiguousarray(arr, dtype=np.float32).tofile(os.path.join(td, f"{name}{i}.bin"))
            t0 = time.perf_counter()
            ps = [subprocess.Popen([orc.REF_BIN, "cpu", "1", "1", str(T_sample), str(D)] +
                                   [os.path.join(td, f"{name}{i}.bin") for name in ("q", "k", "v", "do")] +
                                   [os.path.join(td, f"out{i}")], stdout=subprocess.DEVNULL, cwd=td) for i in range(procs)]
            rcs = [p.wait() for p in ps]
            dt = time.perf_counter() - t0
        if any(rcs):
            raise RuntimeError("oracle/_ref/ref_attention failed")
        return flops / dt / 1e12, "reference", dt
    parts = _cpu_heads(cfg, first_head, procs, T_sample)
    q, k, v, do = (np.stack([p[j] for p in parts])[:, None] for j in range(4))
    t0 = time.perf_counter()
    orc.oracle_f32(q, k, v, do, scale=cfg.scale, threads=procs)
    dt = time.perf_counter() - t0
    return flops / dt / 1e12, "port", dt


def config1_in_full():
    """Configuration 1 (B4 H4 T128 D64 fp32, the one designated for the reference's CPU path) run whole, one process."""
    from oracle import oracle as orc
    from inferno_b200.synth import CONFIGS, make_config_inputs
    c1 = CONFIGS["c1"]
    q, k, v, do = make_config_inputs(c1)
    if orc.have_ref():
        _, _, _, _, tm = orc.ref_attention(q, k, v, do, device="cpu")
        ms, kind = float(tm["fwd_ms"]) + float(tm["bwd_ms"]), "reference"
        extra = dict(fwd_ms=tm["fwd_ms"], bwd_ms=tm["bwd_ms"])
    else:
        t0 = time.perf_counter()
        orc.oracle_f32(q, k, v, do, scale=c1.scale, threads=1)
        ms, kind, extra = 1e3 * (time.perf_counter() - t0), "port", {}
    return dict(workload="c1: B=4 H=4 T=128 d_head=64 fp32, whole configuration, 1 core", ms=ms, kind=kind,
                gflops=c1.flops() / (ms * 1e-3) / 1e9, **extra)


def cpu_baseline_object(cfg, steps: int, with_extras: bool):
    cores = min(host_cores(), 64)
    T_s = min(cfg.T, CPU_SAMPLE_T)
    secs, kind = [], "port"
    for i in range(steps):
        _, kind, dt = cpu_sample(cfg, T_s, cores, first_head=i * cores)
        secs.append(dt)
    value = 7.0 * cores * float(T_s) ** 2 * cfg.D * steps / sum(secs) / 1e12
    obj = dict(value=value, unit=UNIT, cores=cores, kind=kind, seconds=sum(secs),
               sample=f"{steps} pass(es) of {cores} heads, one per host core, each the first {T_s} positions of a T={cfg.T} "
                      f"D={cfg.D} causal head, fp32 (the reference has no bf16)")
    # the whole configuration at this rate (extrapolated linearly in the head count; for a prefix sample also in T^2)
    obj["extrapolated_full_config_seconds"] = cfg.flops() / (value * 1e12)
    if with_extras:
        v1, _, dt1 = cpu_sample(cfg, T_s, 1)
        obj["one_core"] = dict(value=v1, unit=UNIT, cores=1, seconds=dt1, sample=f"one head, first {T_s} positions, one core")
        obj["config1_in_full"] = config1_in_full()
    return obj


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = min(host_cores(), 64)
    T_s = min(cfg.T, CPU_SAMPLE_T)
    kind = "port"
    for i in range(args.warmup):
        _, kind, _ = cpu_sample(cfg, T_s, cores, first_head=i * cores)
    secs = []
    for i in range(args.steps):
        _, kind, dt = cpu_sample(cfg, T_s, cores, first_head=(args.warmup + i) * cores)
        secs.append(dt)
    total_flops = 7.0 * cores * float(T_s) ** 2 * cfg.D * args.steps
    value = total_flops / sum(secs) / 1e12 if secs else 0.0
    sample = (f"{cores} heads per step, one per host core, each the first {T_s} positions of a "
              f"T={cfg.T} D={cfg.D} causal head, fp32 (the reference has no bf16)")
    line = dict(impl="reference", metric=metric_name(cfg), value=value, unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * sum(secs) / max(1, len(secs)), higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                config=workload_config(cfg, args.gpus),
                cpu_baseline=dict(value=value, unit=UNIT, cores=cores, kind=kind, sample=sample),
                e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def ref_cuda_timing(cfg):
    """The reference's own CUDA path (cuBLAS SGEMM + its SIMT scale / mask / softmax kernels, built for sm_100a) on the
    whole configuration, once: the only pre-existing GPU implementation of this path.  Small fp32 configurations only
    (it materialises several [B,H,T,T] matrices)."""
    from oracle import oracle as orc
    from inferno_b200.synth import make_config_inputs
    if not orc.have_ref():
        return dict(unavailable="oracle/_ref/ref_attention is not built")
    if cfg.dtype != "f32" or cfg.B * cfg.H * cfg.T * cfg.T * 4 > (1 << 30):
        return dict(unavailable="configuration too large for the reference's materialised [B,H,T,T] matrices")
    q, k, v, do = make_config_inputs(cfg)
    # two passes in one process, the second reported: the first pays for the context, the cuBLAS handle and first launches
    _, _, _, _, tm = orc.ref_attention(q, k, v, do, device="cuda", reps=2)
    ms = float(tm["fwd_ms"]) + float(tm["bwd_ms"])
    return dict(fwd_ms=tm["fwd_ms"], bwd_ms=tm["bwd_ms"], tflops=cfg.flops() / (ms * 1e-3) / 1e12,
                what="reference CUDA path (composed ops; cuBLAS SGEMM + SIMT kernels), second pass in its process, wall clock around "
                     "forward and around backward including its host<->device copies of the operands' results")


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def generate_shard(cfg, heads, torch, threads: int):
    """Pinned host tensors q, k, v, dO [n, 1, T, D] of this rank's heads, each head from its own stream."""
    import numpy as np
    from inferno_b200.synth import bf16_bits, make_head_inputs
    n, T, D = len(heads), cfg.T, cfg.D
    bf16 = cfg.dtype == "bf16"
    host = [torch.empty((n, 1, T, D), dtype=torch.int16 if bf16 else torch.float32) for _ in range(4)]
    if torch.cuda.is_available():
        host = [h.pin_memory() for h in host]
    views = [h.numpy() for h in host]

    def one(i):
        for j, a in enumerate(make_head_inputs(cfg, heads[i])):
            views[j][i, 0] = bf16_bits(a).view(np.int16) if bf16 else a

    with ThreadPoolExecutor(max(1, threads)) as ex:
        list(ex.map(one, range(n)))
    return [h.view(torch.bfloat16) if bf16 else h for h in host]


def head_checksums(torch, tensors, chunk: int = 32):
    """[n, len(tensors)] int64: per head, sum over elements of bit pattern * (1 + index mod 65521), wrapping."""
    n = tensors[0].shape[0]
    per = tensors[0][0].numel()
    dev = tensors[0].device
    w = (torch.arange(per, device=dev, dtype=torch.int64) % 65521) + 1
    out = torch.empty((n, len(tensors)), dtype=torch.int64, device=dev)
    for j, t in enumerate(tensors):
        bits = t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32).view(n, per)
        for h0 in range(0, n, chunk):
            out[h0:h0 + chunk, j] = (bits[h0:h0 + chunk].to(torch.int64) * w).sum(dim=1)
    return out


def validate(cfg, torch, dist, world, heads, host_in, outs, tol):
    """Outside the timed region: float64 check of the first and last head of this rank's shard, checksums of all."""
    import numpy as np
    from oracle import oracle as orc
    o, dq, dk, dv = outs
    errs = {"O": 0.0, "dQ": 0.0, "dK": 0.0, "dV": 0.0}
    checked = sorted({0, len(heads) - 1})
    for i in checked:
        q, k, v, do = (h[i:i + 1].float().numpy() for h in host_in)            # the very bytes the GPU was given
        refs = orc.attn_fp64(q, k, v, do, scale=cfg.scale)
        for name, x, r in zip(errs, (o, dq, dk, dv), refs):
            errs[name] = max(errs[name], orc.rel_err(x[i:i + 1].float().cpu().numpy(), r))
    dev = o.device
    e = torch.tensor([errs[k] for k in ("O", "dQ", "dK", "dV")], device=dev, dtype=torch.float64)
    sums = head_checksums(torch, (o, dk, dv))
    if world > 1:
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        sizes = [len(r) for r in all_shards(cfg.B * cfg.H, world)]
        pad = max(sizes)
        mine = torch.zeros((pad, 3), dtype=torch.int64, device=dev)
        mine[:len(heads)] = sums
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)                                          # the validation gather: NCCL over NVLink
        sums = torch.cat([g[:s] for g, s in zip(gathered, sizes)])
    digest = hashlib.sha256(sums.cpu().numpy().tobytes()).hexdigest()[:16]
    vals = [float(x) for x in e.tolist()]
    return dict(max_rel_err=dict(zip(("O", "dQ", "dK", "dV"), vals)), tol=tol, ok=bool(max(vals) < tol),
                against="float64 evaluation of the same host operands (oracle.attn_fp64)",
                heads_checked=len(checked) * world, heads_checked_per_rank="first and last of the shard",
                checksum=digest, checksum_heads=int(sums.shape[0]),
                checksum_covers="bit patterns of O, dK, dV of every head, gathered over NCCL (all_gather) in head order; "
                                "dQ is summed by fp32 reductions whose order varies and is covered by the tolerance check")


def all_shards(total, world):
    from inferno_b200.shard import shard_range
    return [shard_range(total, r, world) for r in range(world)]


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
    tdt = torch.bfloat16 if cfg.dtype == "bf16" else torch.float32
    host_in = generate_shard(cfg, heads, torch, threads=max(1, min(16, host_cores() // world)))
    q, k, v, do = (h.to(dev, non_blocking=True) for h in host_in)
    o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty(n, 1, T, device=dev, dtype=torch.float32)
    flush = n * T * D * q.element_size() <= L2_BYTES
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None

    def step():
        A.attention_forward(q, k, v, out=o, lse=lse)
        A.attention_backward(q, k, v, o, do, lse, dq=dq, dk=dk, dv=dv)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    W = max(args.warmup, 3)
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    step()
    w0.record()
    for _ in range(W - 1):
        step()
    w1.record()
    torch.cuda.synchronize()
    A.check_device_status()
    ms_est = max(1e-3, w0.elapsed_time(w1) / max(1, W - 1))
    # untimed steps until the GPU has been under load for min_load_seconds: the board settles into the power state
    # (clock under the power cap) that the timed steps then run in, whatever N and however short a step is
    preload_steps = max(0, int(math.ceil(args.min_load_seconds * 1e3 / ms_est)) - W)

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(K)]
    for row in ev:      # create the underlying CUDA events outside the timed region
        for e in row:
            e.record()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    barrier()
    for _ in range(preload_steps):
        step()
    sampler.start()
    t0.record()
    for i in range(K):
        A.set_timing_events(*ev[i][:4])
        if flush:
            flush_buf.fill_(i & 0xff)
            ev[i][4].record()
        step()
        if flush:
            ev[i][5].record()
    t1.record()
    barrier()
    clocks = sampler.stop()
    A.set_timing_events()
    A.check_device_status()
    ms_total = sum(ev[i][4].elapsed_time(ev[i][5]) for i in range(K)) if flush else t0.elapsed_time(t1)
    fwd_ms = statistics.mean(ev[i][0].elapsed_time(ev[i][1]) for i in range(K))
    bwd_ms = statistics.mean(ev[i][2].elapsed_time(ev[i][3]) for i in range(K))
    mhz = clocks.get("sm_mhz") or 0.0
    t = torch.tensor([ms_total / K, fwd_ms, bwd_ms, -mhz], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, fwd_ms_max, bwd_ms_max, neg_mhz = (float(x) for x in t.tolist())
    clocks["sm_mhz_min_over_ranks"] = -neg_mhz
    total_flops = cfg.flops()
    value = total_flops / (ms_step * 1e-3) / 1e12

    # Small configurations (a step of a few hundred microseconds, five dependent launches): the same step replayed as one
    # CUDA graph, which takes the per-launch gaps out.  Reported beside the stream-launched figure, not instead of it.
    graph = None
    if flush and not args.no_cuda_graph:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                step()                                   # the side stream's own workspace, allocated before the capture
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            step()
        gev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(K)]
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        for i in range(K):
            flush_buf.fill_(i & 0xff)
            gev[i][0].record()
            g.replay()
            gev[i][1].record()
        torch.cuda.synchronize()
        tg = torch.tensor([sum(a.elapsed_time(b) for a, b in gev) / K], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        graph = dict(ms_per_step=float(tg.item()), value=total_flops / (float(tg.item()) * 1e-3) / 1e12, unit=UNIT,
                     what="the same forward + backward captured once into a CUDA graph and replayed (its kernel nodes), L2 flushed between replays")

    validation = None
    if not args.no_validate:
        validation = validate(cfg, torch, dist, world, heads, host_in, (o, dq, dk, dv), 2e-2 if cfg.dtype == "bf16" else 1e-3)

    # ---- end to end: pinned host buffers in, host buffers out, copies inside the timed region ----
    if args.e2e_steps <= 0:      # profiling runs only; a bench line without e2e is not a result
        e2e = None
    else:
        e2e = measure_e2e(args, torch, dist, HostAttention, dev, world, n, T, D, tdt, host_in, (o, dk, dv), barrier, total_flops)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    finish(args, cfg, world, n, T, D, K, W, preload_steps, value, ms_step, fwd_ms_max, bwd_ms_max, clocks, e2e, validation, graph, dist)


def measure_e2e(args, torch, dist, HostAttention, dev, world, n, T, D, tdt, hin, resident, barrier, total_flops):
    hc = args.e2e_heads_per_chunk if args.e2e_heads_per_chunk > 0 else max(1, n // 8)
    hc = max(1, min(n, hc))
    pipe = HostAttention(hc, T, D, tdt, dev, nbuf=args.e2e_nbuf)
    hout = [torch.empty((n, 1, T, D), dtype=tdt).pin_memory() for _ in range(4)]
    pipe.run(*hin, *hout)                      # warm-up (also first touch of the pinned pages)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    Ke = max(1, args.e2e_steps)
    e0.record()
    for _ in range(Ke):
        pipe.run(*hin, *hout, wait=False)
    e1.record()
    barrier()
    # the floor: the same copies over the same buffers and chunks, both directions at once, no kernels, all ranks at once
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pipe.copy_only(*hin, *hout)
    barrier()
    c0.record()
    for _ in range(Ke):
        pipe.copy_only(*hin, *hout)
    c1.record()
    barrier()
    pipe.run(*hin, *hout)                      # leave real results in the host buffers for the check below
    te = torch.tensor([e0.elapsed_time(e1) / Ke, c0.elapsed_time(c1) / Ke], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms, copy_ms = (float(x) for x in te.tolist())
    shard_bytes = n * T * D * hin[0].element_size()
    o, dk, dv = resident
    same = all(torch.equal(h, d.cpu()) for h, d in zip((hout[0], hout[2], hout[3]), (o, dk, dv)))
    return dict(value=total_flops / (e2e_ms * 1e-3) / 1e12, unit=UNIT, ms_per_step=e2e_ms, steps=Ke,
                h2d_bytes_per_step=4 * shard_bytes, d2h_bytes_per_step=4 * shard_bytes,
                heads_per_chunk=hc, chunks_per_rank=(n + hc - 1) // hc, staging_sets=args.e2e_nbuf,
                copy_only_ms=copy_ms, h2d_gbs=4 * shard_bytes / (copy_ms * 1e-3) / 1e9, d2h_gbs=4 * shard_bytes / (copy_ms * 1e-3) / 1e9,
                frac_of_copy_floor=copy_ms / e2e_ms,
                copy_floor="the pipeline's own copies (same pinned buffers, same chunks, both directions concurrently, every rank "
                           "at once) without the kernels; the rates are per rank and per direction, max-over-ranks time",
                api="inferno_b200.host_pipeline.HostAttention.run (pinned host in/out, 3-stream chunked pipeline over the C ABI)",
                outputs_equal_resident=bool(same))


def finish(args, cfg, world, n, T, D, K, W, preload_steps, value, ms_step, fwd_ms_max, bwd_ms_max, clocks, e2e, validation, graph, dist):
    pk = peaks()
    bf16 = cfg.dtype == "bf16"
    mma_per_product = 1 if bf16 else 3
    peak = pk["bf16_sustained"] / mma_per_product
    bwd_flops_rank = 5.0 * n * float(T) ** 2 * D
    achieved = bwd_flops_rank / (bwd_ms_max * 1e-3) / 1e12
    mhz = clocks.get("sm_mhz_min_over_ranks") or clocks.get("sm_mhz")
    e = 2 if bf16 else 4
    hbm_bytes = 13.0 * cfg.B * cfg.H * T * D * e + 16.0 * cfg.B * cfg.H * T
    bwd_kernel = f"attn_bwd_persist_kernel<D={D}>" if bf16 else f"attn_bwd_persist_kernel<D={D}, split-bf16>"
    line = dict(
        metric=metric_name(cfg), value=value, unit=UNIT, n_gpus=world, steps=K, warmup=W, ms_per_step=ms_step,
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16" if bf16 else "f32", data="synthetic",
        config=workload_config(cfg, world),
        per_gpu_tflops=value / world,
        preload=dict(steps=preload_steps, why=f"untimed steps after the warm-up so that the GPU has been under load for "
                                              f"{args.min_load_seconds} s when the {K} timed steps start"),
        clock_normalised=dict(ms_x_mhz=ms_step * mhz if mhz else None,
                              per_gpu_tflops_per_mhz=value / world / mhz if mhz else None,
                              note="ms_per_step x slowest rank's median SM MHz during the timed steps: compares runs taken in different power states"),
        fwd=dict(ms=fwd_ms_max, tflops=2.0 * n * float(T) ** 2 * D / (fwd_ms_max * 1e-3) / 1e12),
        bwd_main=dict(ms=bwd_ms_max, tflops=achieved),
        frac_of_bf16_peak=dict(value=value / world / peak, peak_tflops=peak,
                               of=pk["source"] + " sustained cuBLAS bf16" + ("" if bf16 else " / 3 (three bf16 MMAs per product)"),
                               nominal_frac=value / world / (2250.0 / mma_per_product),
                               **({} if bf16 else {"frac_of_nominal_tf32_peak": value / world / 1100.0})),
        hbm=dict(compulsory_bytes_per_step=hbm_bytes, achieved_gbs=hbm_bytes / (ms_step * 1e-3) / 1e9 / world,
                 frac_of_peak=hbm_bytes / (ms_step * 1e-3) / 1e9 / world / pk["hbm_gbs"], peak_gbs=pk["hbm_gbs"], of=pk["source"],
                 note="13*N*e + 16*BH*T bytes (Q, K, V, dO, O in; O, dQ, dK, dV, lse out; delta pre-pass) over the step time, per GPU: "
                      "far below the HBM rate, i.e. the step is compute-bound"),
        clocks=clocks,
        cuda_graph=graph,
        validation=validation,
        e2e=e2e,
        gpu_launches=(5 if bf16 else 4) * K,
        kernels_per_step=["prepare_header_kernel", "attn_fwd_persist_kernel", "bwd_prepass_kernel", "attn_bwd_persist_kernel", "dq_finish_kernel"] if bf16 else
                         ["split_bf16_kernel", "attn_fwd_persist_kernel", "bwd_prepass_kernel", "attn_bwd_persist_kernel (adds its dQ partials straight into dQ)"],
        roofline=dict(bound="tensor", kernel=bwd_kernel, achieved=achieved, peak=peak,
                      unit="TFLOP/s", frac=achieved / peak, of=pk["source"] + ("" if bf16 else " sustained bf16 / 3: the split schedule issues three bf16 MMAs per product"),
                      algorithmic_flops_per_launch=bwd_flops_rank,
                      traffic=TRAFFIC_BYTES_PER_ELEMENT * n * T * D if (TRAFFIC_BYTES_PER_ELEMENT and bf16 and D == 128) else None,
                      traffic_source="ncu capture of one launch of this kernel on B=2 H=16 T=8192 D=128 (dram__bytes_read.sum + "
                                     "dram__bytes_write.sum), scaled by elements per launch; not measured in this run"),
    )
    if bf16 and D == 128 and mhz:
        # The tile shape's own ceiling: a 64-row query block of the backward moves 288 KB through shared memory (176 KB of MMA
        # operand reads, 32 KB of TMA fills, 16 KB of dS^T, 64 KB of dQ^T staging in and out) for 5 x 2 x 128 x 64 x 128 flop,
        # and an SM's shared memory carries 128 bytes per clock.
        sms, block_flops, block_cycles = 148, 5.0 * 2 * 128 * 64 * 128, 288.0 * 1024 / 128
        ceiling = block_flops * sms * mhz * 1e6 / block_cycles / 1e12
        line["roofline"]["shared_memory_ceiling"] = dict(
            tflops=ceiling, frac=achieved / ceiling,
            note="what this tiling could reach at the sampled SM clock if a block took exactly its 288 KB / (128 B/clk) = 2304 cycles; "
                 "causal-adjusted flops count the two diagonal blocks of an item at half, so 0.97 is the most a T = 4096 run can show")
    if world == 1 and not args.no_cpu_baseline:
        try:
            line["cpu_baseline"] = cpu_baseline_object(cfg, steps=6, with_extras=True)
        except Exception as exc:   # the CPU leg must never take the GPU numbers down with it
            line["cpu_baseline"] = dict(value=None, unit=UNIT, cores=0, kind="port", sample=f"failed: {exc}")
    if world == 1 and args.ref_cuda:
        try:
            line["ref_cuda"] = ref_cuda_timing(cfg)
        except Exception as exc:
            line["ref_cuda"] = dict(unavailable=f"failed: {exc}")
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + write) of one attn_bwd_persist_kernel launch per element of a [heads, T, D] operand, from an ncu
# capture of one launch on B=2 H=16 T=8192 D=128: (410.2 + 226.9) MB over 32 heads x 8192 x 128 elements.  DRAM traffic
# of this kernel is proportional to the elements it touches (each operand is read once from DRAM; re-reads by other
# CTAs of a head hit L2).
TRAFFIC_BYTES_PER_ELEMENT = (410.226688e6 + 226.940928e6) / (32 * 8192 * 128)


def main():
    args = parse_args()
    from inferno_b200.synth import CONFIGS
    cfg = CONFIGS[args.config]
    if cfg.name == "c1":
        raise SystemExit("c1 is a parity case (tests/), not a bench workload")
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
