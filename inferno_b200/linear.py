"""Host-side mirror of the reference's ``Linear`` for the two projections around attention.

``Linear::forward`` in the reference is ``matmul(x, W) + b`` with the weight stored ``[in, out]``
(src/inferno/modules/linear.cpp:19-106); its backward is MMBackward + the bias' sum_to_shape
(src/inferno/gradfn/mmbackward.cpp:36-98).  Here both directions run on the tcgen05 GEMM of
``csrc/linear_gemm.cuh`` through the C ABI (bf16 tensors, fp32 bias and accumulation).
"""
from __future__ import annotations

import torch

from . import _capi


def _check(x: torch.Tensor, name: str):
    if not x.is_cuda:
        raise RuntimeError(f"linear: {name} is not on a CUDA device (there is no CPU path)")
    if x.dtype != torch.bfloat16:
        raise TypeError(f"linear: {name} must be bfloat16")


def linear_forward(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w + bias with x [..., K], w [K, N] (the reference's [in, out] storage), bias [N] fp32."""
    _check(x, "x"); _check(w, "w")
    K, N = w.shape
    x2 = x.reshape(-1, K).contiguous()
    w = w.contiguous()
    y = torch.empty((x2.shape[0], N), dtype=torch.bfloat16, device=x.device)
    b = None if bias is None else bias.to(torch.float32).contiguous()
    with torch.cuda.device(x.device):
        rc = _capi.lib().ib200_linear_fwd(x2.data_ptr(), w.data_ptr(), None if b is None else b.data_ptr(), y.data_ptr(),
                                          x2.shape[0], K, N, torch.cuda.current_stream().cuda_stream)
    if rc != _capi.OK:
        raise _capi.Ib200Error(rc, "ib200_linear_fwd")
    return y.reshape(*x.shape[:-1], N)


def linear_backward(x, w, dy, need_dx=True, need_dw=True, need_db=True):
    K, N = w.shape
    x2, dy2 = x.reshape(-1, K).contiguous(), dy.reshape(-1, N).contiguous()
    M = x2.shape[0]
    dx = torch.empty_like(x2) if need_dx else None
    dw = torch.empty((K, N), dtype=torch.bfloat16, device=x.device) if need_dw else None
    db = torch.empty((N,), dtype=torch.float32, device=x.device) if need_db else None
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(x.device):
        rc = _capi.lib().ib200_linear_bwd(x2.data_ptr(), w.contiguous().data_ptr(), dy2.data_ptr(), ptr(dx), ptr(dw), ptr(db),
                                          M, K, N, torch.cuda.current_stream().cuda_stream)
    if rc != _capi.OK:
        raise _capi.Ib200Error(rc, "ib200_linear_bwd")
    return (None if dx is None else dx.reshape(x.shape)), dw, db


class LinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = None if bias is None else bias.dtype
        return linear_forward(x, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx, dw, db = linear_backward(x, w, dy, ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                     ctx.has_bias and ctx.needs_input_grad[2])
        return dx, dw, (None if db is None else db.to(ctx.bias_dtype))


class Linear(torch.nn.Module):
    """``x @ W + b`` with W stored [in, out] like the reference's Linear; bf16 weight, fp32-accumulated GEMM."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.empty(in_features, out_features))
        self.bias = torch.nn.Parameter(torch.zeros(out_features)) if bias else None
        torch.nn.init.normal_(self.weight, 0.0, 0.02)

    def forward(self, x):
        return LinearFunction.apply(x, self.weight, self.bias)


def _time_shape(M: int, K: int, N: int, iters: int = 20):
    """Forward and backward of one projection on synthetic bf16 data, timed with CUDA events."""
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(K, N, device="cuda", generator=g) / K ** 0.5).to(torch.bfloat16)
    b = torch.randn(N, device="cuda", generator=g)
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    fwd = timed(lambda: linear_forward(x, w, b))
    bwd = timed(lambda: linear_backward(x, w, dy))
    flop = 2.0 * M * K * N
    return dict(M=M, K=K, N=N, fwd_ms=fwd, fwd_tflops=flop / fwd / 1e9, bwd_ms=bwd, bwd_tflops=2 * flop / bwd / 1e9)


if __name__ == "__main__":
    import argparse
    import json

    ap = argparse.ArgumentParser(description="time y = x W + b and its backward (dX, dW, db) on one GPU")
    ap.add_argument("M", type=int, nargs="?", default=16384)
    ap.add_argument("K", type=int, nargs="?", default=768)
    ap.add_argument("N", type=int, nargs="?", default=2304)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    print(json.dumps(_time_shape(a.M, a.K, a.N, a.iters)))
