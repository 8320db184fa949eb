"""Host-side logic: synthetic inputs, bf16 rounding, head sharding (incl. a 2-rank gloo run)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from inferno_b200.shard import shard_range, shard_sizes
from inferno_b200.synth import CONFIGS, bf16_round, make_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_inputs_are_deterministic_and_ordered():
    a = make_inputs(2, 3, 16, 8, 42, 0.5, 0.1)
    b = make_inputs(2, 3, 16, 8, 42, 0.5, 0.1)
    for x, y in zip(a, b):
        assert np.array_equal(x, y) and x.dtype == np.float32 and x.shape == (2, 3, 16, 8)
    assert abs(a[0].std() - 0.5) < 0.05 and abs(a[3].std() - 0.1) < 0.02
    assert not np.array_equal(a[0], a[1])


def test_head_slices_match_the_whole():
    full = make_inputs(2, 4, 8, 16, 9, dtype="bf16")
    part = make_inputs(2, 4, 8, 16, 9, dtype="bf16", heads=slice(3, 6))
    for f, p in zip(full, part):
        assert np.array_equal(f.reshape(8, 1, 8, 16)[3:6], p)


def test_bf16_round_matches_torch():
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32) * 3
    x[:4] = [0.0, -0.0, 1.0, 65504.0]
    ours = bf16_round(x)
    theirs = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(ours, theirs)


def test_config_table_matches_the_benchmark_definition():
    c = CONFIGS["c5"]
    assert (c.B, c.H, c.T, c.D, c.dtype, c.seed) == (64, 16, 4096, 128, "bf16", 4)
    assert CONFIGS["c1"].scale == pytest.approx(0.125)
    # fwd 2*BH*T^2*D, bwd 5*BH*T^2*D (causal-adjusted)
    assert CONFIGS["c3"].flops() == pytest.approx(7 * 32 * 8192 ** 2 * 128)
    assert CONFIGS["c2"].flops(bwd=False) == pytest.approx(2 * 96 * 1024 ** 2 * 64)


@pytest.mark.parametrize("total,world", [(1024, 8), (1024, 1), (96, 8), (7, 4), (3, 8)])
def test_shard_ranges_partition_the_heads(total, world):
    seen = []
    for r in range(world):
        seen.extend(shard_range(total, r, world))
    assert seen == list(range(total))
    sizes = shard_sizes(total, world)
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(total, world, world)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_worker(rank, world, port, ret):
    """Each rank evaluates its own head shard with the CPU oracle; the gathered shards must equal
    the single-process result -- the property the multi-GPU bench relies on (no collective inside
    attention; all_gather only for validation)."""
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, H, T, D, seed = 2, 3, 24, 16, 11
    heads = shard_range(B * H, rank, world)
    q, k, v, do = make_inputs(B, H, T, D, seed, heads=slice(heads.start, heads.stop))
    o, dq, dk, dv = orc.oracle_f32(q, k, v, do, scale=1.0 / np.sqrt(D), threads=1)
    local = torch.from_numpy(np.concatenate([o, dq, dk, dv], axis=1).reshape(len(heads), -1))
    sizes = shard_sizes(B * H, world)
    bufs = [torch.empty(n, local.shape[1]) for n in sizes]
    # all_gather needs equal sizes: pad to the largest shard
    pad = max(sizes)
    padded = torch.zeros(pad, local.shape[1])
    padded[: len(heads)] = local
    gathered = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(gathered, padded)
    if rank == 0:
        whole = torch.cat([g[:n] for g, n in zip(gathered, sizes)])
        qf, kf, vf, dof = make_inputs(B, H, T, D, seed)
        ref = orc.oracle_f32(qf, kf, vf, dof, scale=1.0 / np.sqrt(D), threads=1)
        ref = np.concatenate([r.reshape(B * H, 1, T, D) for r in ref], axis=1).reshape(B * H, -1)
        ret["equal"] = bool(np.array_equal(whole.numpy(), ref))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_reproduces_single_process(oracle_mod):
    import torch.multiprocessing as mp
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_gloo_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get("equal") is True


def _bench_validation(rank, world, port, ret):
    """bench.py's own validation code on CPU tensors: per-head operand streams, float64 spot check, checksum gather."""
    sys.path.insert(0, ROOT)
    import bench
    from inferno_b200.synth import AttnConfig
    from oracle import oracle as orc
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = AttnConfig("tiny", 2, 3, 40, 16, "bf16", 7, 1.0, 0.5)
    heads = shard_range(cfg.B * cfg.H, rank, world)
    host_in = bench.generate_shard(cfg, heads, torch, threads=2)
    q, k, v, do = (h.float().numpy() for h in host_in)
    outs = tuple(torch.from_numpy(a).to(torch.bfloat16) for a in orc.oracle_f32(q, k, v, do, scale=cfg.scale, threads=1))
    val = bench.validate(cfg, torch, dist, world, heads, host_in, outs, 2e-2)
    if rank == 0:
        ret[world] = (val["checksum"], val["ok"], val["checksum_heads"], val["heads_checked"])
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_bench_validation_digest_does_not_depend_on_the_rank_count(oracle_mod):
    """The digest the bench prints covers every head's outputs in head order, so a 2-rank run must print the 1-rank value;
    operands of a head depend on (seed, head) only."""
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    _bench_validation(0, 1, 0, ret)
    mp.spawn(_bench_validation, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret[1][0] == ret[2][0] and ret[1][1] and ret[2][1]
    assert ret[1][2] == ret[2][2] == 6 and ret[2][3] == 4
    from inferno_b200.synth import AttnConfig, make_head_inputs
    cfg = AttnConfig("tiny", 2, 3, 40, 16, "bf16", 7, 1.0, 0.5)
    a, b = make_head_inputs(cfg, 4), make_head_inputs(cfg, 4)
    assert all(np.array_equal(x, y) for x, y in zip(a, b))
    assert not np.array_equal(make_head_inputs(cfg, 3)[0], a[0])


def test_bench_line_carries_the_contract_keys(capsys):
    """The JSON line bench.py prints: every key the measurement contract names is present and consistent (built here from
    made-up timings; no GPU involved)."""
    import json
    import types
    import bench
    from inferno_b200.synth import CONFIGS
    cfg = CONFIGS["c5"]
    args = types.SimpleNamespace(min_load_seconds=2.0, no_cpu_baseline=True, ref_cuda=False)
    clocks = dict(sm_mhz=1560.0, sm_max_mhz=1965.0, reasons=["sw_power_cap"], samples=100, sm_mhz_min_over_ranks=1560.0)
    e2e = dict(value=150.0, unit=bench.UNIT, h2d_bytes_per_step=4 << 30, d2h_bytes_per_step=4 << 30)
    ms_step = 17.9
    value = cfg.flops() / (ms_step * 1e-3) / 1e12
    bench.finish(args, cfg, 1, cfg.B * cfg.H, cfg.T, cfg.D, 20, 5, 100, value, ms_step, 4.2, 12.4, clocks, e2e,
                 dict(ok=True, checksum="0" * 16), None, None)
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "roofline", "validation", "hbm"):
        assert key in line, key
    assert line["steps"] == 20 and line["warmup"] == 5 and line["n_gpus"] == 1 and line["higher_is_better"] is True
    assert line["vs_baseline"] is None and line["dtype"] == "bf16" and "workload" in line["config"] and "model" not in line["config"]
    assert abs(line["value"] * line["ms_per_step"] * 1e-3 * 1e12 - cfg.flops()) / cfg.flops() < 1e-9
    r = line["roofline"]
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-12
    assert abs(r["achieved"] - 5.0 * cfg.B * cfg.H * cfg.T ** 2 * cfg.D / 12.4e-3 / 1e12) < 1e-6
    assert line["gpu_launches"] == 5 * 20 and len(line["kernels_per_step"]) == 5
