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


def _check_like(t: torch.Tensor, q: torch.Tensor, name: str):
    """Caller-supplied output tensors: same shape, dtype and device as q (any strides the kernels can address)."""
    if t.shape != q.shape or t.dtype != q.dtype or t.device != q.device:
        raise ValueError(f"causal_attention: `{name}` must match q in shape, dtype and device")
    return t


def _check_lse(lse: torch.Tensor, q: torch.Tensor):
    """The log-sum-exp vector is addressed densely by the kernels: fp32, contiguous [B, H, T], on q's device."""
    B, H, T, _ = q.shape
    if lse.dtype != torch.float32 or lse.device != q.device or tuple(lse.shape) != (B, H, T) or not lse.is_contiguous():
        raise ValueError("causal_attention: `lse` must be a contiguous float32 [B, H, T] tensor on q's device")
    return lse


def _layout(t: torch.Tensor) -> _capi.Layout:
    """Strides of a [B, H, T, D] tensor (any view whose last axis is contiguous) for the strided entry points."""
    if t.stride(3) != 1:
        raise ValueError("causal_attention: the head-dim axis must be contiguous")
    return _capi.Layout(t.stride(0), t.stride(1), t.stride(2))


def _dense_or_view(t: torch.Tensor) -> torch.Tensor:
    """Use the tensor in place when the kernels can address it (contiguous rows, 16-byte aligned strides);
    otherwise make the dense copy the reference makes with .contiguous()."""
    unit = 16 // t.element_size()
    ok = t.stride(3) == 1 and all(t.stride(a) % unit == 0 and t.stride(a) > 0 for a in (0, 1, 2)) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def empty_bthd(B: int, H: int, T: int, D: int, dtype, device) -> torch.Tensor:
    """A [B, H, T, D] view over [B, T, H, D] memory: what the attention output must look like for
    ``y.transpose(1, 2).reshape(B, T, C)`` to be free (InfernoApp/main.cpp:758-761 pays a copy for it)."""
    return torch.empty((B, T, H, D), dtype=dtype, device=device).transpose(1, 2)


def _raise(rc: int, where: str):
    if rc != _capi.OK:
        raise _capi.Ib200Error(rc, where)


def attention_forward(q, k, v, scale: float | None = None, causal: bool = True, math_mode: int = _capi.MATH_SPLIT_BF16,
                      out=None, lse=None):
    """Launch the forward kernel.  Returns (o [B,H,T,D], lse [B,H,T] fp32).  Asynchronous on the current stream.

    q, k, v (and ``out``) may be arbitrary [B,H,T,D] views with a contiguous last axis -- e.g. slices of a packed
    [B,T,3,H,D] projection, or an output laid out [B,T,H,D] -- and are then read and written in place."""
    B, H, T, D = _check_inputs(q, k, v)
    q, k, v = _dense_or_view(q), _dense_or_view(k), _dense_or_view(v)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dt = _DTYPES[q.dtype]
    o = torch.empty((B, H, T, D), dtype=q.dtype, device=q.device) if out is None else _check_like(out, q, "out")
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device) if lse is None else _check_lse(lse, q)
    ws = _workspace.get(_capi.workspace_bytes(B, H, T, D, dt, _capi.PASS_FWD), q.device)
    lq, lk, lv, lo = _layout(q), _layout(k), _layout(v), _layout(o)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = _capi.lib().ib200_attn_fwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                                lq, lk, lv, lo, B, H, T, D, float(scale), int(bool(causal)), dt, int(math_mode),
                                                ws.data_ptr(), ws.numel(), stream)
    _raise(rc, "ib200_attn_fwd_strided")
    return o, lse


def attention_backward(q, k, v, o, dO, lse, scale: float | None = None, causal: bool = True,
                       math_mode: int = _capi.MATH_SPLIT_BF16, dq=None, dk=None, dv=None):
    """Launch the backward kernels.  Returns (dq, dk, dv).  Asynchronous on the current stream.
    Operands and outputs may be strided views as in ``attention_forward``."""
    B, H, T, D = _check_inputs(q, k, v, o, dO)
    q, k, v, o, dO = (_dense_or_view(t) for t in (q, k, v, o, dO))
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dt = _DTYPES[q.dtype]
    _check_lse(lse, q)
    mk = lambda: torch.empty((B, H, T, D), dtype=q.dtype, device=q.device)
    dq = mk() if dq is None else _check_like(dq, q, "dq")
    dk = mk() if dk is None else _check_like(dk, q, "dk")
    dv = mk() if dv is None else _check_like(dv, q, "dv")
    ws = _workspace.get(_capi.workspace_bytes(B, H, T, D, dt, _capi.PASS_BWD), q.device)
    lays = [_layout(t) for t in (q, k, v, o, dO, dq, dk, dv)]
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = _capi.lib().ib200_attn_bwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dO.data_ptr(),
                                                lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), *lays,
                                                B, H, T, D, float(scale), int(bool(causal)), dt, int(math_mode),
                                                ws.data_ptr(), ws.numel(), stream)
    _raise(rc, "ib200_attn_bwd_strided")
    return dq, dk, dv


def check_device_status(device=None) -> None:
    """Synchronise the current stream and raise if a kernel reported an expired wait.  The status word is sticky:
    one check after any number of forward / backward calls on this stream sees the first failure among them."""
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
    With ``bthd_out`` the output is laid out [B,T,H,D] in memory (returned as a [B,H,T,D] view).  When q, k, v are
    slices of one packed [B,T,3,H,D] buffer the gradients are written into one packed buffer of the same layout,
    so that autograd's accumulation into the projection's gradient needs no scatter-add.
    """

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, math_mode, bthd_out):
        B, H, T, D = q.shape
        out = empty_bthd(B, H, T, D, q.dtype, q.device) if bthd_out else None
        o, lse = attention_forward(q, k, v, scale, causal, math_mode, out=out)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.causal, ctx.math_mode = scale, causal, math_mode
        return o

    @staticmethod
    def backward(ctx, dO):
        q, k, v, o, lse = ctx.saved_tensors
        B, H, T, D = q.shape
        packed = (q.stride() == k.stride() == v.stride() and q.stride(2) == 3 * H * D and q.stride(1) == D and
                  k.data_ptr() - q.data_ptr() == H * D * q.element_size() and v.data_ptr() - k.data_ptr() == H * D * q.element_size())
        if packed:
            g = torch.empty((B, T, 3, H, D), dtype=q.dtype, device=q.device)
            dq, dk, dv = (g[:, :, i].transpose(1, 2) for i in range(3))
            attention_backward(q, k, v, o, dO, lse, ctx.scale, ctx.causal, ctx.math_mode, dq=dq, dk=dk, dv=dv)
        else:
            dq, dk, dv = attention_backward(q, k, v, o, dO, lse, ctx.scale, ctx.causal, ctx.math_mode)
        return dq, dk, dv, None, None, None, None


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
                     math_mode: int = _capi.MATH_SPLIT_BF16, bthd_out: bool = False) -> torch.Tensor:
    """``softmax(mask(q k^T * scale)) v`` with a causal mask; differentiable.  q, k, v: [B,H,T,D] tensors or views."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return AttentionBackward.apply(q, k, v, float(scale), True, int(math_mode), bool(bthd_out))


def causal_attention_packed(qkv: torch.Tensor, num_heads: int, scale: float | None = None,
                            math_mode: int = _capi.MATH_SPLIT_BF16) -> torch.Tensor:
    """Attention straight on the fused projection output: ``qkv`` is [B, T, 3*C] (= [B,T,3,H,D]); returns [B, T, C].
    Replaces slice / contiguous / reshape / transpose / contiguous before the kernels and transpose / contiguous /
    reshape after them (InfernoApp/main.cpp:716-737, 758-761) with stride arithmetic: no copy kernel runs."""
    B, T, C3 = qkv.shape
    C = C3 // 3
    D = C // num_heads
    packed = qkv.view(B, T, 3, num_heads, D)
    q, k, v = (packed[:, :, i].transpose(1, 2) for i in range(3))      # [B,H,T,D] views
    y = causal_attention(q, k, v, scale, math_mode, bthd_out=True)      # [B,H,T,D] view over [B,T,H,D] memory
    return y.transpose(1, 2).reshape(B, T, C)
