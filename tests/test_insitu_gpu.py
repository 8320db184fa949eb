"""Configuration 4 in miniature: the attention op inside a GPT training step (PyTorch harness around it)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_attention_inside_a_training_step_matches_torch_composition():
    from inferno_b200.insitu_gpt import GPT, train_step
    torch.manual_seed(0)
    dev = torch.device("cuda")
    cfg = dict(vocab=512, T=256, C=128, H=2, layers=2)     # d_head = 64
    ours = GPT(attn_impl="ib200", **cfg).to(dev).to(torch.bfloat16)
    ref = GPT(attn_impl="torch", **cfg).to(dev).to(torch.bfloat16)
    ref.load_state_dict(ours.state_dict())
    idx = torch.randint(0, cfg["vocab"], (2, cfg["T"]), device=dev)
    tgt = torch.randint(0, cfg["vocab"], (2, cfg["T"]), device=dev)
    losses, grads = [], []
    for m in (ours, ref):
        logits = m(idx)
        loss = torch.nn.functional.cross_entropy(logits.float().view(-1, cfg["vocab"]), tgt.view(-1))
        loss.backward()
        losses.append(float(loss.detach()))
        grads.append(torch.cat([p.grad.float().flatten() for p in m.blocks[0].wqkv.parameters()]))
    assert abs(losses[0] - losses[1]) < 2e-2
    rel = (grads[0] - grads[1]).norm() / grads[1].norm()
    assert rel < 5e-2, f"Wqkv gradient differs by {rel:.3e}"     # bf16 everywhere: tolerance of the bf16 tests plus the MLP path
    opt = torch.optim.AdamW(ours.parameters(), lr=3e-4)
    l0 = float(train_step(ours, opt, idx, tgt).detach())
    for _ in range(20):
        l1 = float(train_step(ours, opt, idx, tgt).detach())
    assert l1 < l0                                             # it trains


def test_insitu_timing_harness_runs():
    from inferno_b200.insitu_gpt import run
    out = run(layers=2, C=256, H=4, vocab=1024, T=512, B=2, steps=2, warmup=1)
    assert out["attn_fwd_ms"] > 0 and out["attn_bwd_main_ms"] > 0 and 0 < out["attn_share_of_step"] < 1


def test_full_variant_matches_torch_composition():
    """Packed attention plus the library's own projection GEMMs inside the model, against the plain PyTorch composition
    with the same weights: loss, and the gradient of the first block's Wqkv (which has passed through W_out's backward,
    the packed attention backward and Wqkv's own weight-gradient GEMM)."""
    from inferno_b200.insitu_gpt import GPT
    torch.manual_seed(1)
    dev = torch.device("cuda")
    cfg = dict(vocab=512, T=256, C=128, H=2, layers=2)
    full = GPT(attn_impl="ib200_full", **cfg).to(dev).to(torch.bfloat16)
    ref = GPT(attn_impl="torch", **cfg).to(dev).to(torch.bfloat16)
    sd = full.state_dict()
    for name in list(sd):          # this library's Linear stores its weight [in, out] (as the reference does), torch's [out, in]
        if name.endswith(("wqkv.weight", "wout.weight")):
            sd[name] = sd[name].t().contiguous()
    ref.load_state_dict(sd)
    idx = torch.randint(0, cfg["vocab"], (2, cfg["T"]), device=dev)
    tgt = torch.randint(0, cfg["vocab"], (2, cfg["T"]), device=dev)
    losses, grads = [], []
    for m in (full, ref):
        loss = torch.nn.functional.cross_entropy(m(idx).float().view(-1, cfg["vocab"]), tgt.view(-1))
        loss.backward()
        losses.append(float(loss.detach()))
        g = m.blocks[0].wqkv.weight.grad.float()
        grads.append(g if m is full else g.t())
    assert abs(losses[0] - losses[1]) < 2e-2
    rel = (grads[0] - grads[1]).norm() / grads[1].norm()
    assert rel < 5e-2, f"Wqkv gradient differs by {rel:.3e}"


def test_full_variant_trains():
    """Packed attention plus the library's own projection GEMMs inside the training step."""
    from inferno_b200.insitu_gpt import GPT, train_step
    torch.manual_seed(0)
    dev = torch.device("cuda")
    m = GPT(vocab=512, T=256, C=128, H=2, layers=2, attn_impl="ib200_full").to(dev).to(torch.bfloat16)
    idx = torch.randint(0, 512, (2, 256), device=dev)
    tgt = torch.randint(0, 512, (2, 256), device=dev)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-4)
    l0 = float(train_step(m, opt, idx, tgt).detach())
    for _ in range(20):
        l1 = float(train_step(m, opt, idx, tgt).detach())
    assert l1 < l0
