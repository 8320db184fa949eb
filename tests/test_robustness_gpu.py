"""Error reporting of the kernels on a GPU, without provoking any fault.

* the bounded-wait path: a self-test kernel waits on a barrier nothing signals, gives up after a millisecond, records
  its site code, frees its tensor memory and exits normally; the host sees IB200_ERR_DEVICE_TIMEOUT once, and the
  attention kernels run correctly afterwards;
* the status word is sticky across calls that share a workspace (a failure recorded before a forward call is still
  there after it);
* the built-in status word used by the entry points that have no caller workspace;
* the range-checked build of the library (every TMA coordinate, tensor-memory address and swizzled store checked on
  the device) passes the small-shape parity cases with a clean status.
"""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

from inferno_b200 import _capi
from inferno_b200 import attention as A
from inferno_b200.synth import make_inputs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _check(ws):
    code = ctypes.c_int(-1)
    rc = _capi.lib().ib200_attn_check(ws.data_ptr(), torch.cuda.current_stream().cuda_stream, ctypes.byref(code))
    return rc, code.value


def _small_parity(oracle_mod, seed=5):
    q, k, v, do = make_inputs(1, 2, 200, 128, seed, 1.0, 0.5, "bf16")
    tq, tk, tv, tdo = (torch.from_numpy(a).cuda().to(torch.bfloat16) for a in (q, k, v, do))
    o, lse = A.attention_forward(tq, tk, tv)
    dq, dk, dv = A.attention_backward(tq, tk, tv, o, tdo, lse)
    torch.cuda.synchronize()
    for x, r in zip((o, dq, dk, dv), oracle_mod.oracle_f32(q, k, v, do)):
        assert oracle_mod.rel_err(x.float().cpu().numpy(), r) < 2e-2


def test_expired_wait_is_reported_once_and_the_gpu_stays_usable(oracle_mod):
    L = _capi.lib()
    ws = torch.randint(0, 255, (4096,), device="cuda", dtype=torch.uint8)      # an uninitialised workspace holds anything
    s = torch.cuda.current_stream().cuda_stream
    assert _check(ws) == (_capi.OK, 0)                                         # garbage is not a status
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert L.ib200_selftest_wait_expiry(ws.data_ptr(), ws.numel(), 1000, s) == _capi.OK
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 500.0                                         # gave up after ~1 ms, not after the 4 s product limit
    assert _check(ws) == (_capi.ERR_DEVICE_TIMEOUT, 190)
    assert _check(ws) == (_capi.OK, 0)                                         # reported once
    _small_parity(oracle_mod)                                                  # tensor memory was released: the kernels still run
    A.check_device_status()


def test_status_word_survives_later_calls_on_the_same_workspace(oracle_mod):
    """A failure recorded in a workspace is still reported after further forward / backward calls have used it."""
    L = _capi.lib()
    _small_parity(oracle_mod)                       # makes sure the per-stream workspace exists and is large enough
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = A._workspace._bufs[(dev.index, torch.cuda.current_stream(dev).cuda_stream)]
    s = torch.cuda.current_stream().cuda_stream
    assert L.ib200_selftest_wait_expiry(ws.data_ptr(), ws.numel(), 500, s) == _capi.OK
    _small_parity(oracle_mod, seed=6)               # forward + backward on the same workspace
    with pytest.raises(_capi.Ib200Error, match="190"):
        A.check_device_status()
    A.check_device_status()                         # cleared by the report


def test_builtin_status_word_after_projection_calls():
    from inferno_b200 import linear
    x = torch.randn(256, 128, device="cuda").to(torch.bfloat16)
    w = torch.randn(128, 256, device="cuda").to(torch.bfloat16)
    y = linear.linear_forward(x, w, None)
    code = ctypes.c_int(-1)
    rc = _capi.lib().ib200_attn_check_static(torch.cuda.current_stream().cuda_stream, ctypes.byref(code))
    assert (rc, code.value) == (_capi.OK, 0)
    ref = x.float() @ w.float()
    assert float((y.float() - ref).norm() / ref.norm()) < 1e-2


_BOUNDS_SCRIPT = r"""
import ctypes, sys, numpy as np, torch
from inferno_b200 import _capi, attention as A
from inferno_b200.synth import make_inputs
from oracle import oracle as orc
assert "bounds" in _capi.lib()._name
cases = [(1, 2, 200, 64, "f32", 1e-3), (2, 1, 128, 64, "f32", 1e-3), (1, 2, 320, 128, "bf16", 2e-2), (2, 3, 500, 64, "bf16", 2e-2),
         (1, 1, 1, 64, "bf16", 2e-2), (1, 40, 700, 128, "bf16", 2e-2)]
for (B, H, T, D, dt, tol) in cases:
    q, k, v, do = make_inputs(B, H, T, D, 11, 1.0, 0.5, dt)
    tdt = torch.float32 if dt == "f32" else torch.bfloat16
    tq, tk, tv, tdo = (torch.from_numpy(a).cuda().to(tdt) for a in (q, k, v, do))
    o, lse = A.attention_forward(tq, tk, tv)
    dq, dk, dv = A.attention_backward(tq, tk, tv, o, tdo, lse)
    A.check_device_status()          # raises on a recorded range violation (codes 201-208) or an expired wait
    for name, x, r in zip("O dQ dK dV".split(), (o, dq, dk, dv), orc.oracle_f32(q, k, v, do)):
        err = orc.rel_err(x.float().cpu().numpy(), r)
        assert err < tol, (B, H, T, D, dt, name, err)
x = torch.randn(512, 256, device="cuda").to(torch.bfloat16); w = torch.randn(256, 384, device="cuda").to(torch.bfloat16)
y = torch.empty(512, 384, device="cuda", dtype=torch.bfloat16)
assert _capi.lib().ib200_linear_fwd(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 512, 256, 384, torch.cuda.current_stream().cuda_stream) == 0
code = ctypes.c_int(-1)
assert _capi.lib().ib200_attn_check_static(torch.cuda.current_stream().cuda_stream, ctypes.byref(code)) == 0 and code.value == 0
ref = x.float() @ w.float()
assert float((y.float() - ref).norm() / ref.norm()) < 1e-2
print("bounds-checked build: all cases clean")
"""


def test_range_checked_build_runs_the_small_shapes_clean(oracle_mod):
    from inferno_b200 import build
    env = dict(os.environ, IB200_LIB=build.build(bounds=True), PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-c", _BOUNDS_SCRIPT], env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "all cases clean" in res.stdout
