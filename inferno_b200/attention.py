"""Host-side mirror of the reference's operator idiom for the fused attention op.

In the reference an op is a free function ``Inferno::op(const Tensor&...) -> Tensor`` that
checks devices and shapes, allocates the output, switches on the device type, calls the
CUDA launcher with raw pointers, and attaches a backward node when gradients are enabled
(src/inferno/core/ops.cpp:204-270; nodes: src/inferno/gradfn/node.h:23-45).  The fused op
stands where InfernoApp/main.cpp:737-754 composes matmul / scale / mask / Softmax / matmul:

    y = causal_attention(q, k, v, scale)         # q, k, v: dense [B, H, T, D] on a CUDA device

Here the tensor type is ``torch.Tensor`` (device memory, streams), the launcher is the C ABI
of ``include/inferno_b200_attn.h`` reached through ctypes, and the backward node is a
``torch.autograd.Function``.  There is no CPU arm: a CPU tensor is rejected, exactly as the
library itself refuses to run without an sm_100 device.
"""
from __future__ import annotations

import math

import torch

from . import _capi

_DTYPES = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16}


class _Workspace:
    """Caller-owned scratch, cached per (device, stream) and grown on demand."""

    def __init__(self):
        self._bufs = {}

    def get(self, nbytes: int, device: torch.device) -> torch.Tensor:
        key = (device.index, torch.cuda.current_stream(device).cuda_stream)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
            self._bufs[key] = buf
        return buf


_workspace = _Workspace()


def _check_inputs(*tensors: torch.Tensor):
    q = tensors[0]
    if q.dim() != 4:
        raise ValueError("causal_attention expects [B, H, T, D] tensors")
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("causal_attention: tensor is not on a CUDA device (there is no CPU path)")
        if t.device != q.device:
            raise RuntimeError("causal_attention: tensors are on different devices")
        if t.dtype != q.dtype or t.dtype not in _DTYPES:
            raise TypeError("causal_attention: dtype must be float32 or bfloat16, the same for all tensors")
        if t.shape != q.shape:
            raise ValueError("causal_attention: q, k, v (and dO) must have the same shape")
    return q.shape


def _raise(rc: int, where: str):
    if rc != _capi.OK:
        raise _capi.Ib200Error(rc, where)


def attention_forward(q, k, v, scale: float | None = None, causal: bool = True, math_mode: int = _capi.MATH_TF32,
                      out=None, lse=None):
    """Launch the forward kernel.  Returns (o [B,H,T,D], lse [B,H,T] fp32).  Asynchronous on the current stream."""
    B, H, T, D = _check_inputs(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dt = _DTYPES[q.dtype]
    o = torch.empty_like(q) if out is None else out
    if lse is None:
        lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    ws = _workspace.get(_capi.workspace_bytes(B, H, T, D, dt, _capi.PASS_FWD), q.device)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = _capi.lib().ib200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                        B, H, T, D, float(scale), int(bool(causal)), dt, int(math_mode),
                                        ws.data_ptr(), ws.numel(), stream)
    _raise(rc, "ib200_attn_fwd")
    return o, lse


def attention_backward(q, k, v, o, dO, lse, scale: float | None = None, causal: bool = True,
                       math_mode: int = _capi.MATH_TF32, dq=None, dk=None, dv=None):
    """Launch the backward kernels.  Returns (dq, dk, dv).  Asynchronous on the current stream."""
    B, H, T, D = _check_inputs(q, k, v, o, dO)
    q, k, v, o, dO = (t.contiguous() for t in (q, k, v, o, dO))
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dt = _DTYPES[q.dtype]
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(q) if dk is None else dk
    dv = torch.empty_like(q) if dv is None else dv
    ws = _workspace.get(_capi.workspace_bytes(B, H, T, D, dt, _capi.PASS_BWD), q.device)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = _capi.lib().ib200_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dO.data_ptr(),
                                        lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                        B, H, T, D, float(scale), int(bool(causal)), dt, int(math_mode),
                                        ws.data_ptr(), ws.numel(), stream)
    _raise(rc, "ib200_attn_bwd")
    return dq, dk, dv


def check_device_status(device=None) -> None:
    """Synchronise the current stream and raise if a kernel reported an expired wait."""
    import ctypes
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspace._bufs.get(key)
    if buf is None:
        return
    code = ctypes.c_int(0)
    with torch.cuda.device(device):
        rc = _capi.lib().ib200_attn_check(buf.data_ptr(), torch.cuda.current_stream().cuda_stream, ctypes.byref(code))
    if rc != _capi.OK:
        raise _capi.Ib200Error(rc, f"ib200_attn_check (device code {code.value})")


def set_timing_events(fwd_start=None, fwd_stop=None, bwd_start=None, bwd_stop=None) -> None:
    """Have later calls on this thread record these ``torch.cuda.Event``s (timing enabled, created on the
    current device) right around the forward / backward main kernels.  No arguments switches it off."""
    handles = []
    for ev in (fwd_start, fwd_stop, bwd_start, bwd_stop):
        if ev is None:
            handles.append(None)
        else:
            if not ev.cuda_event:          # torch creates the event lazily, on first record
                ev.record()
            handles.append(ev.cuda_event)
    _raise(_capi.lib().ib200_attn_set_timing_events(*handles), "ib200_attn_set_timing_events")


class AttentionBackward(torch.autograd.Function):
    """The backward node of the fused op: saves q, k, v, out and lse; produces dq, dk, dv.

    Plays the role a ``class AttentionBackward : public Node`` would in the reference
    (src/inferno/gradfn/node.h:23-45: ``backward()``, ``release()``, ``get_inputs()``).
    """

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, math_mode):
        o, lse = attention_forward(q, k, v, scale, causal, math_mode)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.causal, ctx.math_mode = scale, causal, math_mode
        return o

    @staticmethod
    def backward(ctx, dO):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, o, dO, lse, ctx.scale, ctx.causal, ctx.math_mode)
        return dq, dk, dv, None, None, None


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
                     math_mode: int = _capi.MATH_TF32) -> torch.Tensor:
    """``softmax(mask(q k^T * scale)) v`` with a causal mask; differentiable."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return AttentionBackward.apply(q, k, v, float(scale), True, int(math_mode))
