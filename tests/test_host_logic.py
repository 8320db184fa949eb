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
