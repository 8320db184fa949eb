"""Operands that live inside larger buffers (packed [B,T,3,H,D] projections, [B,T,H,D] outputs): the strided entry
points must give exactly what the dense ones give on dense copies of the same values."""
import pytest
import torch

from inferno_b200 import attention as A
from inferno_b200.synth import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,H,T,D,dt", [(2, 3, 200, 64, torch.bfloat16), (1, 2, 320, 128, torch.bfloat16), (2, 2, 130, 64, torch.float32)])
def test_packed_qkv_and_bthd_output_match_dense(B, H, T, D, dt):
    name = "bf16" if dt == torch.bfloat16 else "f32"
    q, k, v, do = (torch.from_numpy(a).cuda().to(dt) for a in make_inputs(B, H, T, D, 77, 1.0, 0.5, name))
    # dense reference run
    o_ref, lse_ref = A.attention_forward(q, k, v)
    g_ref = A.attention_backward(q, k, v, o_ref, do, lse_ref)
    # the same values inside a packed [B,T,3,H,D] buffer; outputs laid out [B,T,H,D]; dO given as [B,T,H,D] too
    packed = torch.stack([t.transpose(1, 2) for t in (q, k, v)], dim=2).contiguous()          # [B,T,3,H,D]
    qs, ks, vs = (packed[:, :, i].transpose(1, 2) for i in range(3))
    assert not qs.is_contiguous() and qs.stride(2) == 3 * H * D
    o = A.empty_bthd(B, H, T, D, dt, q.device)
    o2, lse2 = A.attention_forward(qs, ks, vs, out=o)
    do_s = do.transpose(1, 2).contiguous().transpose(1, 2)
    gpacked = torch.empty_like(packed)
    dq, dk, dv = (gpacked[:, :, i].transpose(1, 2) for i in range(3))
    A.attention_backward(qs, ks, vs, o2, do_s, lse2, dq=dq, dk=dk, dv=dv)
    torch.cuda.synchronize()
    A.check_device_status()
    assert torch.equal(o2, o_ref) and torch.equal(lse2, lse_ref)
    assert o2.transpose(1, 2).is_contiguous()                       # [B,T,H,D] memory: reshape to [B,T,C] is free
    assert torch.equal(dk, g_ref[1]) and torch.equal(dv, g_ref[2])
    assert (dq.float() - g_ref[0].float()).norm() / g_ref[0].float().norm() < 1e-3


def test_packed_autograd_path_matches_dense_autograd_path():
    B, H, T, D = 2, 4, 256, 64
    C = H * D
    torch.manual_seed(5)
    qkv = torch.randn(B, T, 3 * C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(B, T, C, device="cuda", dtype=torch.bfloat16)
    y = A.causal_attention_packed(qkv, H)
    y.backward(gy)
    g_packed = qkv.grad.clone()
    qkv.grad = None
    q, k, v = (t.reshape(B, T, H, D).transpose(1, 2).contiguous() for t in qkv.split(C, dim=2))
    y2 = A.causal_attention(q, k, v).transpose(1, 2).reshape(B, T, C)
    y2.backward(gy)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    rel = (g_packed.float() - qkv.grad.float()).norm() / qkv.grad.float().norm()
    assert rel < 1e-3


def test_misaligned_strides_are_rejected_or_copied():
    # a token stride that is not a multiple of 16 bytes cannot be described to the TMA unit: the host mirror
    # falls back to the dense copy the reference would make, and the raw C ABI refuses it
    import ctypes
    from inferno_b200 import _capi
    B, H, T, D = 1, 1, 64, 64
    buf = torch.randn(B, H, T, D + 4, device="cuda", dtype=torch.bfloat16)
    q = buf[..., :D]
    o, _ = A.attention_forward(q, q, q)          # copied internally
    o_ref, _ = A.attention_forward(q.contiguous(), q.contiguous(), q.contiguous())
    assert torch.equal(o, o_ref)
    lay = _capi.Layout(H * T * (D + 4), T * (D + 4), D + 4)
    ws = torch.empty(4096, device="cuda", dtype=torch.uint8)
    lse = torch.empty(B, H, T, device="cuda")
    rc = _capi.lib().ib200_attn_fwd_strided(q.data_ptr(), q.data_ptr(), q.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                            ctypes.byref(lay), None, None, None, B, H, T, D, 0.125, 1, _capi.DTYPE_BF16, 0,
                                            ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == _capi.ERR_MISALIGNED


@pytest.mark.parametrize("B,H,T,D", [(2, 3, 200, 64), (1, 4, 320, 128)])
def test_packed_autograd_path_against_the_oracle(oracle_mod, B, H, T, D):
    """`causal_attention_packed` on a [B, T, 3*H*D] projection output, checked directly against the float64 evaluation:
    the output [B, T, C] and the gradient with respect to the packed buffer."""
    import numpy as np
    from inferno_b200.synth import bf16_round
    rng = np.random.default_rng(77 + T)
    qkv_np = bf16_round(rng.standard_normal((B, T, 3, H, D), dtype=np.float32))
    dy_np = bf16_round(0.5 * rng.standard_normal((B, T, H, D), dtype=np.float32))
    qkv = torch.from_numpy(qkv_np.reshape(B, T, 3 * H * D)).cuda().to(torch.bfloat16).requires_grad_(True)
    y = A.causal_attention_packed(qkv, H)
    y.backward(torch.from_numpy(dy_np.reshape(B, T, H * D)).cuda().to(torch.bfloat16))
    torch.cuda.synchronize()
    A.check_device_status()
    q, k, v = (np.ascontiguousarray(qkv_np[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))      # [B,H,T,D]
    do = np.ascontiguousarray(dy_np.transpose(0, 2, 1, 3))
    o, dq, dk, dv = oracle_mod.attn_fp64(q, k, v, do)
    got_y = y.detach().float().cpu().numpy().reshape(B, T, H, D).transpose(0, 2, 1, 3)
    got_g = qkv.grad.float().cpu().numpy().reshape(B, T, 3, H, D)
    assert oracle_mod.rel_err(got_y, o) < 2e-2
    for i, ref in enumerate((dq, dk, dv)):
        assert oracle_mod.rel_err(got_g[:, :, i].transpose(0, 2, 1, 3), ref) < 2e-2
