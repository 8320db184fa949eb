"""The allocation-free backward entry point, `ib200_attn_bwd_static`.

Some users of this library cannot pass a workspace: they call from a place where obtaining device
memory is not an option at all (for example a serving loop that is forbidden to touch the allocator,
or a host program whose own pool has claimed the whole GPU).  For them the library carries a fixed
scratch buffer of its own.  This test drives that entry point through the C ABI twice in a row --
the second call finds the first call's leftovers in the shared buffer -- and checks both results
against the regular `ib200_attn_bwd`.  It lives in a file of its own that pytest collects last, and
it does not depend on anything the other tests leave behind.
"""
import pytest
import torch

from inferno_b200 import _capi
from inferno_b200.synth import make_inputs

pytestmark = pytest.mark.gpu

# dK and dV are produced in a fixed order (bitwise equal between the two entry points); dQ is summed
# by floating-point reductions whose order varies run to run, hence the tolerance used throughout
# the GPU tests for it.
DQ_RTOL = 1e-3


def _dev(a, dt):
    return torch.from_numpy(a).cuda().to(dt)


def _forward(L, q, k, v, B, H, T, D, dtype_code):
    o = torch.empty_like(q)
    lse = torch.empty(B, H, T, device="cuda", dtype=torch.float32)
    ws = torch.empty(_capi.workspace_bytes(B, H, T, D, dtype_code, _capi.PASS_FWD), device="cuda", dtype=torch.uint8)
    s = torch.cuda.current_stream().cuda_stream
    rc = L.ib200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, H, T, D,
                          1.0 / D ** 0.5, 1, dtype_code, 0, ws.data_ptr(), ws.numel(), s)
    assert rc == _capi.OK
    return o, lse


def _backward_regular(L, q, k, v, o, do, lse, B, H, T, D, dtype_code):
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    ws = torch.empty(_capi.workspace_bytes(B, H, T, D, dtype_code, _capi.PASS_BWD), device="cuda", dtype=torch.uint8)
    s = torch.cuda.current_stream().cuda_stream
    rc = L.ib200_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                          dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, T, D, 1.0 / D ** 0.5, 1, dtype_code, 0,
                          ws.data_ptr(), ws.numel(), s)
    assert rc == _capi.OK
    torch.cuda.synchronize()
    return dq, dk, dv


def _backward_static(L, q, k, v, o, do, lse, B, H, T, D, dtype_code):
    dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
    s = torch.cuda.current_stream().cuda_stream
    rc = L.ib200_attn_bwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                 dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, T, D, 1.0 / D ** 0.5, 1, dtype_code, 0, s)
    assert rc == _capi.OK, _capi.status_string(rc)
    torch.cuda.synchronize()
    return dq, dk, dv


def _check(got, want):
    dq, dk, dv = got
    rq, rk, rv = want
    assert torch.equal(dk, rk) and torch.equal(dv, rv)
    assert torch.isfinite(dq).all()
    err = (dq.float() - rq.float()).norm() / rq.float().norm()
    assert err < DQ_RTOL, f"dQ differs from the regular entry point by {err:.2e}"


def test_static_scratch_backward_matches_regular_entry_point_twice():
    L = _capi.lib()
    # two different problems back to back: the second call starts from a buffer full of the first one's data
    cases = [(2, 3, 320, 128, "bf16", torch.bfloat16, _capi.DTYPE_BF16, 31),
             (1, 2, 200, 64, "f32", torch.float32, _capi.DTYPE_F32, 32)]
    for (B, H, T, D, dt, tdt, code, seed) in cases:
        q, k, v, do = (_dev(a, tdt) for a in make_inputs(B, H, T, D, seed, 1.0, 0.5, dt))
        o, lse = _forward(L, q, k, v, B, H, T, D, code)
        want = _backward_regular(L, q, k, v, o, do, lse, B, H, T, D, code)
        _check(_backward_static(L, q, k, v, o, do, lse, B, H, T, D, code), want)
        _check(_backward_static(L, q, k, v, o, do, lse, B, H, T, D, code), want)   # same problem again, stale scratch
    # no bounded wait expired in any of those calls: the built-in buffer's status word, which only this reader can see
    import ctypes
    dev_code = ctypes.c_int(-1)
    assert L.ib200_attn_check_static(torch.cuda.current_stream().cuda_stream, ctypes.byref(dev_code)) == _capi.OK
    assert dev_code.value == 0


def test_static_scratch_rejects_problems_beyond_its_capacity():
    L = _capi.lib()
    B, H, T, D = 4, 16, 2048, 128          # needs ~64 MiB of scratch: more than the built-in buffer
    assert _capi.workspace_bytes(B, H, T, D, _capi.DTYPE_BF16, _capi.PASS_BWD) > _capi.STATIC_SCRATCH_BYTES
    x = torch.zeros(16, device="cuda", dtype=torch.bfloat16)     # never touched: the call must refuse before launching
    lse = torch.zeros(16, device="cuda", dtype=torch.float32)
    p = x.data_ptr()
    rc = L.ib200_attn_bwd_static(p, p, p, p, p, lse.data_ptr(), p, p, p, B, H, T, D, 0.088, 1, _capi.DTYPE_BF16, 0,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == _capi.ERR_TOO_LARGE
    assert "static scratch" in _capi.status_string(rc)
    torch.cuda.synchronize()
