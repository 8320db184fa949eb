"""Attention forward + backward for operands that live in host memory.

This is the reference's own usage pattern made explicit: its ``Tensor`` constructor copies a host
vector to the device (``src/inferno/core/tensorimpl.cpp:24-61``: cudaMalloc + synchronous
cudaMemcpy) and results come back with ``Tensor::to(cpu)`` (``src/inferno/core/tensor.cpp:609-693``).
Here the same round trip is chunked over heads and pipelined on three streams -- host-to-device
copies, kernels, device-to-host copies -- with double-buffered device staging, so that the copies
of one chunk overlap the kernels of another.  A staging set's input half is released as soon as the
kernels have consumed it and its output half once the results have left, so neither copy direction
ever waits for the other.  Heads are independent, so chunking changes nothing.
"""
from __future__ import annotations

import torch

from . import attention as A


class HostAttention:
    def __init__(self, heads_per_chunk: int, T: int, D: int, dtype: torch.dtype, device, nbuf: int = 2):
        self.hc, self.T, self.D, self.dtype = heads_per_chunk, T, D, dtype
        self.device = torch.device(device)
        self.nbuf = nbuf
        mk = lambda: torch.empty((heads_per_chunk, 1, T, D), dtype=dtype, device=self.device)
        self.bufs = [dict(q=mk(), k=mk(), v=mk(), do=mk(), o=mk(), dq=mk(), dk=mk(), dv=mk(),
                          lse=torch.empty((heads_per_chunk, 1, T), dtype=torch.float32, device=self.device))
                     for _ in range(nbuf)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)

    def run(self, q, k, v, do, o, dq, dk, dv) -> None:
        """All arguments: pinned host tensors [heads, 1, T, D] (or any shape with that many elements per
        head).  Returns after every output has landed in host memory."""
        heads = q.shape[0]
        main = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(main)
        in_free = [None] * self.nbuf      # kernels of the chunk that last used this set have read its inputs
        out_free = [None] * self.nbuf     # results of that chunk have been copied out of this set
        for ci, h0 in enumerate(range(0, heads, self.hc)):
            n = min(self.hc, heads - h0)
            b = self.bufs[ci % self.nbuf]
            with torch.cuda.stream(self.s_in):
                if in_free[ci % self.nbuf] is not None:
                    self.s_in.wait_event(in_free[ci % self.nbuf])
                for name, src in (("q", q), ("k", k), ("v", v), ("do", do)):
                    b[name][:n].copy_(src[h0:h0 + n], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ev_in)
                if out_free[ci % self.nbuf] is not None:
                    self.s_run.wait_event(out_free[ci % self.nbuf])
                A.attention_forward(b["q"][:n], b["k"][:n], b["v"][:n], out=b["o"][:n], lse=b["lse"][:n])
                A.attention_backward(b["q"][:n], b["k"][:n], b["v"][:n], b["o"][:n], b["do"][:n], b["lse"][:n],
                                     dq=b["dq"][:n], dk=b["dk"][:n], dv=b["dv"][:n])
                ev_run = torch.cuda.Event()
                ev_run.record(self.s_run)
                in_free[ci % self.nbuf] = ev_run
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_run)
                for name, dst in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
                    dst[h0:h0 + n].copy_(b[name][:n], non_blocking=True)
                ev_out = torch.cuda.Event()
                ev_out.record(self.s_out)
                out_free[ci % self.nbuf] = ev_out
        for s in (self.s_in, self.s_run, self.s_out):
            main.wait_stream(s)
