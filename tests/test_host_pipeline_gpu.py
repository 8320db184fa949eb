"""The pinned-host pipeline (inferno_b200.host_pipeline.HostAttention): operands in host memory, chunked over heads on
three streams with two staging sets.  Its results must equal, bit for bit, those of the same kernels run on resident
tensors, for every head of every chunk, also when the last chunk is short and when the pipeline object is reused."""
import pytest
import torch

from inferno_b200 import attention as A
from inferno_b200.host_pipeline import HostAttention

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("heads,hc,T,D", [(10, 3, 256, 128), (7, 2, 200, 64), (4, 8, 128, 128)])
def test_pipeline_matches_resident_path(heads, hc, T, D):
    g = torch.Generator().manual_seed(heads * 1000 + T)
    hin = [torch.randn((heads, 1, T, D), generator=g).to(torch.bfloat16).pin_memory() for _ in range(4)]
    hout = [torch.empty((heads, 1, T, D), dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    pipe = HostAttention(hc, T, D, torch.bfloat16, "cuda")
    for _ in range(3):                                   # reuse: staging sets and events of the previous run
        for t in hout:
            t.fill_(float("nan"))
        pipe.run(*hin, *hout)
        torch.cuda.synchronize()
        q, k, v, do = (t.cuda() for t in hin)
        o, lse = A.attention_forward(q, k, v)
        dq, dk, dv = A.attention_backward(q, k, v, o, do, lse)
        torch.cuda.synchronize()
        # dQ goes through fp32 atomics whose order is not fixed, so it is compared to a tolerance; the rest bitwise
        assert torch.equal(hout[0], o.cpu())
        assert torch.equal(hout[2], dk.cpu()) and torch.equal(hout[3], dv.cpu())
        assert float((hout[1].float() - dq.cpu().float()).abs().max()) <= 1e-2 * float(dq.float().abs().max())
