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
        # one event per staging set and pipeline stage, created once: a run records and waits, it creates nothing
        self.ev_in = [torch.cuda.Event() for _ in range(nbuf)]
        self.ev_run = [torch.cuda.Event() for _ in range(nbuf)]
        self.ev_out = [torch.cuda.Event() for _ in range(nbuf)]
        self.ev_done = torch.cuda.Event()

    def run(self, q, k, v, do, o, dq, dk, dv, wait: bool = True) -> None:
        """All arguments: pinned host tensors [heads, 1, T, D] (or any shape with that many elements per head).
        With ``wait`` (the default) the call returns after every output has landed in host memory; with
        ``wait=False`` the results are only ordered on the caller's current stream, and the host must synchronise
        that stream (or call ``wait_done``) before it reads the output tensors."""
        heads = q.shape[0]
        main = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(main)
        used = [False] * self.nbuf
        for ci, h0 in enumerate(range(0, heads, self.hc)):
            n = min(self.hc, heads - h0)
            j = ci % self.nbuf
            b = self.bufs[j]
            with torch.cuda.stream(self.s_in):
                if used[j]:
                    self.s_in.wait_event(self.ev_run[j])       # the kernels of the chunk that last used this set have read its inputs
                for name, src in (("q", q), ("k", k), ("v", v), ("do", do)):
                    b[name][:n].copy_(src[h0:h0 + n], non_blocking=True)
                self.ev_in[j].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[j])
                if used[j]:
                    self.s_run.wait_event(self.ev_out[j])      # the results of that chunk have been copied out of this set
                A.attention_forward(b["q"][:n], b["k"][:n], b["v"][:n], out=b["o"][:n], lse=b["lse"][:n])
                A.attention_backward(b["q"][:n], b["k"][:n], b["v"][:n], b["o"][:n], b["do"][:n], b["lse"][:n],
                                     dq=b["dq"][:n], dk=b["dk"][:n], dv=b["dv"][:n])
                self.ev_run[j].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[j])
                for name, dst in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
                    dst[h0:h0 + n].copy_(b[name][:n], non_blocking=True)
                self.ev_out[j].record(self.s_out)
            used[j] = True
        for s in (self.s_in, self.s_run, self.s_out):
            main.wait_stream(s)
        self.ev_done.record(main)
        if wait:
            self.ev_done.synchronize()

    def wait_done(self) -> None:
        """Block the host until the last ``run`` has delivered its outputs."""
        self.ev_done.synchronize()

    def copy_only(self, q, k, v, do, o, dq, dk, dv) -> None:
        """The copies of ``run`` without its kernels: the same chunks over the same pinned buffers, host-to-device
        and device-to-host concurrently on the two copy streams.  What this takes is the floor ``run`` is measured
        against (asynchronous; synchronise the current stream afterwards)."""
        heads = q.shape[0]
        main = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_out):
            s.wait_stream(main)
        for ci, h0 in enumerate(range(0, heads, self.hc)):
            n = min(self.hc, heads - h0)
            b = self.bufs[ci % self.nbuf]
            with torch.cuda.stream(self.s_in):
                for name, src in (("q", q), ("k", k), ("v", v), ("do", do)):
                    b[name][:n].copy_(src[h0:h0 + n], non_blocking=True)
            with torch.cuda.stream(self.s_out):
                for name, dst in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
                    dst[h0:h0 + n].copy_(b[name][:n], non_blocking=True)
        for s in (self.s_in, self.s_out):
            main.wait_stream(s)
