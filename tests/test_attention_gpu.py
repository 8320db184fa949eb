"""Parity of the CUDA kernels, called through the C ABI, against the CPU checkers.

Tolerances (normwise relative error ||x - ref||_F / ||ref||_F on O, dQ, dK, dV):
    fp32 I/O : 1e-3      bf16 I/O : 2e-2
The reference path itself has no bf16; for bf16 cases the checkers consume the bf16-rounded
inputs upcast to fp32.
"""

import numpy as np
import pytest
import torch

from inferno_b200 import _capi
from inferno_b200 import attention as A
from inferno_b200.synth import CONFIGS, make_config_inputs, make_inputs

pytestmark = pytest.mark.gpu

TOL = {"f32": 1e-3, "bf16": 2e-2}
TDT = {"f32": torch.float32, "bf16": torch.bfloat16}
from golden_cases import MANIFEST, load_case


def run_gpu(q, k, v, do, dt, causal=True):
    tq, tk, tv, tdo = (torch.from_numpy(a).cuda().to(TDT[dt]) for a in (q, k, v, do))
    o, lse = A.attention_forward(tq, tk, tv, causal=causal)
    dq, dk, dv = A.attention_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    torch.cuda.synchronize()
    A.check_device_status()
    return [t.float().cpu().numpy() for t in (o, dq, dk, dv)], lse.cpu().numpy()


def assert_close(outs, refs, tol, orc, what=""):
    for name, x, r in zip(("O", "dQ", "dK", "dV"), outs, refs):
        err = orc.rel_err(x, r)
        assert np.isfinite(x).all(), f"{what} {name} has non-finite values"
        assert err < tol, f"{what} {name}: rel err {err:.3e} >= {tol}"


@pytest.mark.parametrize("name", [n for n in sorted(MANIFEST) if MANIFEST[n]["D"] in (64, 128)])
def test_golden_vectors(oracle_mod, name):
    """Outputs of the reference's own code, stored under tests/golden/."""
    c, (q, k, v, do), gold = load_case(name)
    outs, _ = run_gpu(q, k, v, do, c["dtype"])
    if c["T"] == 1:
        # dQ = dK = 0 exactly in the reference; a relative error is undefined, so compare absolutely
        tol = TOL[c["dtype"]]
        assert oracle_mod.rel_err(outs[0], gold["o"]) < tol and oracle_mod.rel_err(outs[3], gold["dv"]) < tol
        assert np.abs(outs[1]).max() < 1e-3 and np.abs(outs[2]).max() < 1e-3
        return
    assert_close(outs, [gold[k_] for k_ in ("o", "dq", "dk", "dv")], TOL[c["dtype"]], oracle_mod, name)


def test_config1_against_reference_restatement(oracle_mod):
    """B4 H4 T128 D64 fp32, seed 0: the configuration the reference runs on its CPU path."""
    cfg = CONFIGS["c1"]
    q, k, v, do = make_config_inputs(cfg)
    refs = oracle_mod.oracle_f32(q, k, v, do)
    outs, lse = run_gpu(q, k, v, do, "f32")
    assert_close(outs, refs, TOL["f32"], oracle_mod, "c1")
    lse64 = oracle_mod.attn_fp64(q, k, v, want_lse=True)[-1]
    assert np.abs(lse - lse64).max() < 1e-4


def test_config2_head_subsample(oracle_mod):
    """GPT-2-small shape, fp32 I/O: all 96 heads run on the GPU, 6 of them are checked
    against the reference restatement (C, ~1 s per head) and all finite."""
    cfg = CONFIGS["c2"]
    q, k, v, do = make_config_inputs(cfg)
    outs, _ = run_gpu(q, k, v, do, "f32")
    sel = [0, 13, 47, 95, 50, 71]
    flat = lambda a: a.reshape(cfg.B * cfg.H, 1, cfg.T, cfg.D)[sel]
    refs = oracle_mod.oracle_f32(flat(q), flat(k), flat(v), flat(do), scale=cfg.scale)
    assert_close([flat(x) for x in outs], refs, TOL["f32"], oracle_mod, "c2")
    assert all(np.isfinite(x).all() for x in outs)


@pytest.mark.parametrize("shape", [
    (1, 1, 1, 128), (1, 3, 63, 128), (1, 2, 65, 64), (2, 1, 129, 128), (1, 2, 257, 64),
    (1, 1, 300, 128), (3, 1, 128, 64), (1, 5, 448, 128), (1, 2, 1000, 64),
])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_ragged_and_edge_shapes(oracle_mod, shape, dt):
    B, H, T, D = shape
    if dt == "f32" and D != 64:
        pytest.skip("fp32 I/O is built for head dim 64 (the reference's fp32 configurations)")
    q, k, v, do = make_inputs(B, H, T, D, 100 + T, 1.0, 1.0, dt)
    refs = oracle_mod.attn_fp64(q, k, v, do)
    outs, _ = run_gpu(q, k, v, do, dt)
    if T == 1:
        assert oracle_mod.rel_err(outs[0], v) < TOL[dt] and oracle_mod.rel_err(outs[3], do) < TOL[dt]
        assert np.abs(outs[1]).max() < 1e-3 and np.abs(outs[2]).max() < 1e-3
        return
    assert_close(outs, refs, TOL[dt], oracle_mod, str(shape))


def test_non_causal_mode(oracle_mod):
    B, H, T, D = 1, 2, 200, 64
    q, k, v, do = make_inputs(B, H, T, D, 5, dtype="bf16")
    outs, _ = run_gpu(q, k, v, do, "bf16", causal=False)
    q64, k64, v64, do64 = (a.astype(np.float64) for a in (q, k, v, do))
    s = np.einsum("bhtd,bhsd->bhts", q64, k64) / np.sqrt(D)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    o = p @ v64
    dp = np.einsum("bhtd,bhsd->bhts", do64, v64)
    ds = p * (dp - (dp * p).sum(-1, keepdims=True)) / np.sqrt(D)
    refs = [o, ds @ k64, np.swapaxes(ds, -1, -2) @ q64, np.swapaxes(p, -1, -2) @ do64]
    assert_close(outs, refs, TOL["bf16"], oracle_mod, "non-causal")


def test_config3_long_context_subsample_and_properties(oracle_mod):
    """B2 H16 T8192 D128 bf16 at full size: two heads against the fp64 evaluator, every head
    through size-independent properties (causality, batch permutation, finiteness)."""
    cfg = CONFIGS["c3"]
    g = torch.Generator(device="cuda").manual_seed(cfg.seed)
    mk = lambda std: (torch.randn(cfg.B, cfg.H, cfg.T, cfg.D, device="cuda", generator=g) * std).to(torch.bfloat16)
    q, k, v, do = mk(0.5), mk(0.5), mk(0.5), mk(0.1)
    o, lse = A.attention_forward(q, k, v)
    dq, dk, dv = A.attention_backward(q, k, v, o, do, lse)
    torch.cuda.synchronize()
    A.check_device_status()
    for t in (o, dq, dk, dv, lse):
        assert torch.isfinite(t).all()
    for (b, h) in ((0, 3), (1, 15)):
        sl = lambda t: t[b:b + 1, h:h + 1].float().cpu().numpy()
        refs = oracle_mod.attn_fp64(sl(q), sl(k), sl(v), sl(do))
        assert_close([sl(o), sl(dq), sl(dk), sl(dv)], refs, TOL["bf16"], oracle_mod, f"c3 head {b},{h}")
    # causality: changing keys/values at positions >= 4096 cannot change rows < 4096 (bitwise)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 4096:] += 1
    v2[:, :, 4096:] -= 1
    o2, lse2 = A.attention_forward(q, k2, v2)
    assert torch.equal(o[:, :, :4096], o2[:, :, :4096]) and torch.equal(lse[:, :, :4096], lse2[:, :, :4096])
    assert not torch.equal(o[:, :, 4096:], o2[:, :, 4096:])
    # heads are independent: permuting the batch permutes the outputs (bitwise for O, dK, dV)
    perm = torch.tensor([1, 0], device="cuda")
    o3, lse3 = A.attention_forward(q[perm].contiguous(), k[perm].contiguous(), v[perm].contiguous())
    dq3, dk3, dv3 = A.attention_backward(q[perm].contiguous(), k[perm].contiguous(), v[perm].contiguous(), o3,
                                         do[perm].contiguous(), lse3)
    assert torch.equal(o3, o[perm]) and torch.equal(dk3, dk[perm]) and torch.equal(dv3, dv[perm])
    # dQ is accumulated with floating-point atomics: order-dependent rounding only
    assert (dq3.float() - dq[perm].float()).norm() / dq.float().norm() < 1e-3
    # the last key receives gradient from the last query only
    p_last = torch.exp((q[:, :, -1].float() * k[:, :, -1].float()).sum(-1) * cfg.scale - lse[:, :, -1])
    want = p_last[..., None] * do[:, :, -1].float()
    assert (dv[:, :, -1].float() - want).norm() / want.norm() < 2e-2


def test_config5_shape_replicated_heads(oracle_mod):
    """T4096 D128 bf16 with many heads (a 1/8 shard of the box-scale configuration: 128 heads):
    every head is a copy of one of 4 prototypes, so each output must equal its prototype's
    (bitwise for O, dK, dV) and the prototypes are checked against fp64."""
    cfg = CONFIGS["c5"]
    heads, T, D = 128, cfg.T, cfg.D
    pq, pk, pv, pdo = (torch.from_numpy(a).cuda().to(torch.bfloat16)
                       for a in make_inputs(4, 1, T, D, cfg.seed, cfg.qkv_std, cfg.do_std, "bf16"))
    rep = lambda t: t.reshape(4, T, D).repeat(heads // 4, 1, 1).reshape(heads, 1, T, D).contiguous()
    q, k, v, do = rep(pq), rep(pk), rep(pv), rep(pdo)
    o, lse = A.attention_forward(q, k, v)
    dq, dk, dv = A.attention_backward(q, k, v, o, do, lse)
    torch.cuda.synchronize()
    A.check_device_status()
    for t in (o, dk, dv):
        assert torch.equal(t.reshape(heads // 4, 4, T, D), t[:4].reshape(1, 4, T, D).expand(heads // 4, 4, T, D))
    spread = (dq.reshape(heads // 4, 4, T, D).float() - dq[:4].reshape(1, 4, T, D).float()).norm() / dq.float().norm()
    assert spread < 1e-3
    np_ = lambda t: t[:2].float().cpu().numpy()
    refs = oracle_mod.attn_fp64(np_(q), np_(k), np_(v), np_(do))
    assert_close([np_(o), np_(dq), np_(dk), np_(dv)], refs, TOL["bf16"], oracle_mod, "c5 prototypes")


@pytest.mark.parametrize("dt,D", [("bf16", 128), ("bf16", 64), ("f32", 64)])
def test_linearity_in_dO_and_causal_prefix_at_bench_length(dt, D):
    """Size-independent properties at T = 4096 (the bench's sequence length), no checker needed.
    (1) The backward is linear in dO: with 2 * dO every partial product doubles exactly (a power of two commutes with every
        rounding), so dK and dV double bit for bit, and dQ up to the order of its floating-point reduction.
    (2) A causal prefix is a self-contained sub-problem: O and lse of the first 2048 positions, computed from a T = 2048
        call, equal the first 2048 rows of the T = 4096 call bit for bit (the same tiles are walked in the same order)."""
    B, H, T = 2, 3, 4096
    q, k, v, do = (torch.from_numpy(a).cuda().to(TDT[dt]) for a in make_inputs(B, H, T, D, 55, 1.0, 0.25, dt))
    o, lse = A.attention_forward(q, k, v)
    dq, dk, dv = A.attention_backward(q, k, v, o, do, lse)
    dq2, dk2, dv2 = A.attention_backward(q, k, v, o, do * 2, lse)
    torch.cuda.synchronize()
    A.check_device_status()
    assert torch.equal(dk2, dk * 2) and torch.equal(dv2, dv * 2)
    assert (dq2.float() - 2 * dq.float()).norm() / dq.float().norm() < 1e-3
    Tp = 2048
    op, lsep = A.attention_forward(q[:, :, :Tp].contiguous(), k[:, :, :Tp].contiguous(), v[:, :, :Tp].contiguous())
    torch.cuda.synchronize()
    assert torch.equal(op, o[:, :, :Tp]) and torch.equal(lsep, lse[:, :, :Tp])


def _torch_fp32_reference(q, k, v, do):
    """Causal attention and its gradients in plain fp32 torch ops on the GPU (scores materialised)."""
    q, k, v, do = (t.float() for t in (q, k, v, do))
    T, D = q.shape[-2], q.shape[-1]
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    s = (q @ k.transpose(-1, -2)) / D ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, device=q.device, dtype=torch.bool), 1), float("-inf"))
    o = torch.softmax(s, -1) @ v
    o.backward(do)
    return o.detach(), q.grad, k.grad, v.grad


def test_random_shapes_and_item_counts():
    """bf16 kernels walk a list of work items with one CTA per SM, drawing items from a counter: shapes with fewer items
    than SMs, one more or one less than a whole round, many light heads, and seeded random (B, H, T, D); every output
    against fp32 torch ops, and O / dK / dV bitwise equal between two runs (dQ is a floating-point reduction)."""
    import random
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rng = random.Random(7)
    shapes = [(1, 2, 129, 128), (sms, 1, 128, 128), (sms + 1, 1, 128, 64), (sms - 1, 1, 256, 128), (37, 4, 256, 128),
              (2, 74, 384, 64), (3, 50, 257, 128), (1, 1, 2048, 64)]
    shapes += [(rng.randint(1, 6), rng.randint(1, 6), rng.randint(2, 1500), rng.choice([64, 128])) for _ in range(24)]
    g = torch.Generator(device="cuda").manual_seed(11)
    for (B, H, T, D) in shapes:
        q, k, v = (torch.randn(B, H, T, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
        do = (torch.randn(B, H, T, D, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        o, lse = A.attention_forward(q, k, v)
        grads = A.attention_backward(q, k, v, o, do, lse)
        o2, lse2 = A.attention_forward(q, k, v)
        grads2 = A.attention_backward(q, k, v, o2, do, lse2)
        torch.cuda.synchronize()
        A.check_device_status()
        assert torch.equal(o, o2) and torch.equal(grads[1], grads2[1]) and torch.equal(grads[2], grads2[2]), (B, H, T, D)
        for name, x, r in zip(("O", "dQ", "dK", "dV"), (o,) + tuple(grads), _torch_fp32_reference(q, k, v, do)):
            err = ((x.float() - r).norm() / r.norm()).item()
            assert err < TOL["bf16"], f"{(B, H, T, D)} {name}: rel err {err:.3e}"


def test_backward_is_linear_in_dO():
    q, k, v, do = (torch.from_numpy(a).cuda().to(torch.bfloat16) for a in make_inputs(1, 2, 512, 128, 8, dtype="bf16"))
    o, lse = A.attention_forward(q, k, v)
    g1 = A.attention_backward(q, k, v, o, do, lse)
    g2 = A.attention_backward(q, k, v, o, (do * 2).contiguous(), lse)
    torch.cuda.synchronize()
    # doubling dO is exact in bf16, so dK and dV double exactly; dQ up to atomic ordering
    assert torch.equal(g2[1].float(), g1[1].float() * 2) and torch.equal(g2[2].float(), g1[2].float() * 2)
    assert (g2[0].float() - 2 * g1[0].float()).norm() / g2[0].float().norm() < 1e-3


def test_forward_is_bitwise_repeatable():
    q, k, v, _ = (torch.from_numpy(a).cuda().to(torch.bfloat16) for a in make_inputs(2, 2, 1024, 128, 9, dtype="bf16"))
    o1, l1 = A.attention_forward(q, k, v)
    o2, l2 = A.attention_forward(q, k, v)
    torch.cuda.synchronize()
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


def test_autograd_function_matches_explicit_calls():
    q, k, v, do = (torch.from_numpy(a).cuda().to(torch.bfloat16).requires_grad_(True)
                   for a in make_inputs(1, 2, 256, 64, 10, dtype="bf16"))
    y = A.causal_attention(q, k, v)
    y.backward(do.detach())
    o, lse = A.attention_forward(q.detach(), k.detach(), v.detach())
    dq, dk, dv = A.attention_backward(q.detach(), k.detach(), v.detach(), o, do.detach(), lse)
    torch.cuda.synchronize()
    assert torch.equal(y.detach(), o) and torch.equal(k.grad, dk) and torch.equal(v.grad, dv)
    assert (q.grad.float() - dq.float()).norm() / dq.float().norm() < 1e-3


def test_abi_errors_on_gpu():
    """Argument errors are reported as status codes through the C ABI with a device present."""
    L = _capi.lib()
    q = torch.zeros(1, 1, 64, 64, device="cuda", dtype=torch.bfloat16)
    lse = torch.zeros(1, 1, 64, device="cuda")
    ws = torch.zeros(4096, device="cuda", dtype=torch.uint8)
    s = torch.cuda.current_stream().cuda_stream
    ok = L.ib200_attn_fwd(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), lse.data_ptr(), 1, 1, 64, 64, 0.125, 1,
                          _capi.DTYPE_BF16, 0, ws.data_ptr(), ws.numel(), s)
    assert ok == _capi.OK
    bad = L.ib200_attn_fwd(q.data_ptr() + 2, q.data_ptr(), q.data_ptr(), q.data_ptr(), lse.data_ptr(), 1, 1, 64, 64, 0.125, 1,
                           _capi.DTYPE_BF16, 0, ws.data_ptr(), ws.numel(), s)
    assert bad == _capi.ERR_MISALIGNED
    small = L.ib200_attn_bwd(*([q.data_ptr()] * 5), lse.data_ptr(), *([q.data_ptr()] * 3), 1, 1, 64, 64, 0.125, 1,
                             _capi.DTYPE_BF16, 0, ws.data_ptr(), 1024, s)
    assert small == _capi.ERR_WORKSPACE
    torch.cuda.synchronize()
    import ctypes
    code = ctypes.c_int(-1)
    assert L.ib200_attn_check(ws.data_ptr(), s, ctypes.byref(code)) == _capi.OK and code.value == 0
