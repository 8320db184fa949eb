"""Configuration 4: attention forward + backward timed in situ inside a full training step of a 12-layer GPT.

The model mirrors the topology of the reference's application (InfernoApp/main.cpp:828-1035): token
embedding + sinusoidal positional encoding, pre-LayerNorm transformer blocks (ln1 -> attention -> +x ->
ln2 -> Linear 4x -> tanh-GELU -> Linear -> +x), final LayerNorm, untied output head, cross-entropy loss,
AdamW (lr 3e-4, betas (0.9, 0.95), weight decay 0.1: include/inferno/optim/adamw.h:15-22).  Everything
around attention is PyTorch library code and is only the harness; the attention sub-path -- the part this
repository replaces -- is `inferno_b200.attention.causal_attention`.  Attention is timed with CUDA events
placed by the library's timing hook right around its main kernels, while the whole step runs.

    python -m inferno_b200.insitu_gpt [--layers 12 --d-model 768 --heads 12 --vocab 8192 --T 1024 --B 16 --steps 5]
"""
from __future__ import annotations

import argparse
import json
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import attention as A
from . import linear as L


def sinusoidal_pe(T: int, C: int, device) -> torch.Tensor:
    pos = torch.arange(T, device=device, dtype=torch.float32)[:, None]
    div = torch.exp(torch.arange(0, C, 2, device=device, dtype=torch.float32) * (-math.log(10000.0) / C))
    pe = torch.zeros(T, C, device=device)
    pe[:, 0::2] = torch.sin(pos * div)
    pe[:, 1::2] = torch.cos(pos * div)
    return pe


class Block(nn.Module):
    def __init__(self, C: int, H: int, attn_impl: str):
        super().__init__()
        self.H, self.attn_impl = H, attn_impl
        self.ln1, self.ln2 = nn.LayerNorm(C), nn.LayerNorm(C)
        if attn_impl == "ib200_full":      # projections on this library's tcgen05 GEMM too (weights stored [in, out] like the reference)
            self.wqkv, self.wout = L.Linear(C, 3 * C), L.Linear(C, C)
        else:
            self.wqkv, self.wout = nn.Linear(C, 3 * C), nn.Linear(C, C)
        self.ff1, self.ff2 = nn.Linear(C, 4 * C), nn.Linear(4 * C, C)

    def attention(self, x: torch.Tensor) -> torch.Tensor:
        B, T, C = x.shape
        if self.attn_impl in ("ib200_packed", "ib200_full"):
            # the kernels read q, k, v in place inside the projection output and write [B,T,H,D]: no layout copies
            return self.wout(A.causal_attention_packed(self.wqkv(x), self.H))
        q, k, v = self.wqkv(x).split(C, dim=2)
        q, k, v = (t.reshape(B, T, self.H, C // self.H).transpose(1, 2).contiguous() for t in (q, k, v))   # [B,H,T,D]
        if self.attn_impl == "ib200":
            y = A.causal_attention(q, k, v)
        else:  # plain PyTorch composition of the same math, fp32 softmax: the in-situ cross-check
            s = (q.float() @ k.float().transpose(-1, -2)) / math.sqrt(q.shape[-1])
            s = s.masked_fill(torch.triu(torch.ones(T, T, device=x.device, dtype=torch.bool), 1), float("-inf"))
            y = (torch.softmax(s, -1) @ v.float()).to(q.dtype)
        return self.wout(y.transpose(1, 2).reshape(B, T, C))

    def forward(self, x):
        x = x + self.attention(self.ln1(x))
        return x + self.ff2(F.gelu(self.ff1(self.ln2(x)), approximate="tanh"))


class GPT(nn.Module):
    def __init__(self, vocab: int, T: int, C: int, H: int, layers: int, attn_impl: str = "ib200"):
        super().__init__()
        self.emb = nn.Embedding(vocab, C)
        self.blocks = nn.ModuleList(Block(C, H, attn_impl) for _ in range(layers))
        self.ln_f, self.head = nn.LayerNorm(C), nn.Linear(C, vocab)
        self.T = T
        for p in self.parameters():            # random-init weights N(0, 0.02)
            if p.dim() >= 2:
                nn.init.normal_(p, 0.0, 0.02)

    def forward(self, idx):
        x = self.emb(idx) + sinusoidal_pe(idx.shape[1], self.emb.embedding_dim, idx.device).to(self.emb.weight.dtype)
        for b in self.blocks:
            x = b(x)
        return self.head(self.ln_f(x))


def train_step(model, opt, idx, tgt):
    logits = model(idx)
    loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), tgt.view(-1))
    opt.zero_grad(set_to_none=True)
    loss.backward()
    opt.step()
    return loss


def run(layers=12, C=768, H=12, vocab=8192, T=1024, B=16, steps=5, warmup=3, seed=3, attn_impl="ib200"):
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(seed)
    model = GPT(vocab, T, C, H, layers, attn_impl).to(dev).to(torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator(device=dev).manual_seed(seed)
    idx = torch.randint(0, vocab, (B, T), device=dev, generator=g)
    tgt = torch.randint(0, vocab, (B, T), device=dev, generator=g)
    for _ in range(warmup):
        train_step(model, opt, idx, tgt)
    # One event quadruple per layer: the hook records around the main kernels of each attention call.  The forward
    # calls run in layer order and the backward calls in reverse, so each call needs its own events.
    fwd_ms, bwd_ms, step_ms = [], [], []
    for _ in range(steps):
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(layers)]
        for row in evs:
            for e in row:
                e.record()
        calls = {"f": 0, "b": 0}
        orig_f, orig_b = A.attention_forward, A.attention_backward

        def fwd_hook(*a, **kw):
            i = calls["f"]; calls["f"] += 1
            A.set_timing_events(evs[i][0], evs[i][1], None, None)
            try:
                return orig_f(*a, **kw)
            finally:
                A.set_timing_events()          # the hook is per host thread: switch it off where it was switched on

        def bwd_hook(*a, **kw):
            i = layers - 1 - calls["b"]; calls["b"] += 1
            A.set_timing_events(None, None, evs[i][2], evs[i][3])
            try:
                return orig_b(*a, **kw)       # runs on autograd's worker thread
            finally:
                A.set_timing_events()

        A.attention_forward, A.attention_backward = fwd_hook, bwd_hook
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        try:
            t0.record()
            loss = train_step(model, opt, idx, tgt)
            t1.record()
            torch.cuda.synchronize()
        finally:
            A.attention_forward, A.attention_backward = orig_f, orig_b
            A.set_timing_events()
        fwd_ms.append(sum(r[0].elapsed_time(r[1]) for r in evs))
        bwd_ms.append(sum(r[2].elapsed_time(r[3]) for r in evs))
        step_ms.append(t0.elapsed_time(t1))
    A.check_device_status()
    D = C // H
    unit = B * H * float(T) ** 2 * D * layers
    f, b, s = (sorted(x)[len(x) // 2] for x in (fwd_ms, bwd_ms, step_ms))
    return dict(config=dict(layers=layers, d_model=C, heads=H, d_head=D, vocab=vocab, T=T, B=B, dtype="bf16", attn_impl=attn_impl),
                loss=float(loss.detach()), step_ms=s, attn_fwd_ms=f, attn_bwd_main_ms=b,
                attn_fwd_tflops=2 * unit / (f * 1e-3) / 1e12, attn_bwd_tflops=5 * unit / (b * 1e-3) / 1e12,
                attn_share_of_step=(f + b) / s)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12); ap.add_argument("--d-model", type=int, default=768)
    ap.add_argument("--heads", type=int, default=12); ap.add_argument("--vocab", type=int, default=8192)
    ap.add_argument("--T", type=int, default=1024); ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--attn", default="ib200", choices=["ib200", "ib200_packed", "ib200_full"],
                    help="ib200: dense [B,H,T,D] operands (the reference's layout copies stay); ib200_packed: operands read in place; ib200_full: packed attention plus this library's GEMM for Wqkv / W_out")
    a = ap.parse_args()
    print(json.dumps(run(a.layers, a.d_model, a.heads, a.vocab, a.T, a.B, a.steps, attn_impl=a.attn)))
