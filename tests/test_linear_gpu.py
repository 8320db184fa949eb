"""The projection GEMM (bf16 tcgen05, fp32 accumulate, bias epilogue) against a float32 PyTorch matmul.
Tolerance: normwise relative error 1e-2 (bf16 output rounding is 2^-9 per element)."""
import pytest
import torch

from inferno_b200 import _capi
from inferno_b200 import linear as L

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (256, 768, 2304), (1000, 768, 768), (136, 72, 264), (4096, 3072, 768),
                                   (8192, 256, 256),     # weight gradient: 2 output tiles, split-K over 8 slabs
                                   (128, 8192, 256)])    # forward: 1 output tile, split-K with the bias going in once
def test_forward_and_backward_match_float32_reference(M, K, N):
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(K, N, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device="cuda", generator=g)
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    y = L.linear_forward(x, w, b)
    dx, dw, db = L.linear_backward(x, w, dy)
    torch.cuda.synchronize()
    xf, wf, dyf = x.float(), w.float(), dy.float()
    assert rel(y, xf @ wf + b) < 1e-2
    assert rel(dx, dyf @ wf.t()) < 1e-2
    assert rel(dw, xf.t() @ dyf) < 1e-2
    assert rel(db, dyf.sum(0)) < 1e-4


def test_generic_entry_point_all_operand_majors():
    M, N, K = 256, 512, 192
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    want = a.float() @ b.float()
    lib = _capi.lib()
    s = torch.cuda.current_stream().cuda_stream
    for a_t in (0, 1):
        for b_t in (0, 1):
            aa = a.t().contiguous() if a_t else a
            bb = b.t().contiguous() if b_t else b
            c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            rc = lib.ib200_gemm_bf16(aa.data_ptr(), bb.data_ptr(), c.data_ptr(), None, M, N, K, a_t, b_t, s)
            assert rc == _capi.OK
            torch.cuda.synchronize()
            assert rel(c, want) < 1e-2, (a_t, b_t)
    assert lib.ib200_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), None, M, N, 100, 0, 0, s) == _capi.ERR_UNSUPPORTED
    assert lib.ib200_gemm_bf16(None, b.data_ptr(), c.data_ptr(), None, M, N, K, 0, 0, s) == _capi.ERR_INVALID_ARGUMENT


def test_linear_module_autograd():
    torch.manual_seed(1)
    lin = L.Linear(256, 384).cuda().to(torch.bfloat16)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    y.backward(torch.ones_like(y))
    ref = x.detach().float() @ lin.weight.detach().float() + lin.bias.detach().float()
    assert rel(y.detach(), ref) < 1e-2
    assert rel(lin.bias.grad, torch.full((384,), 4 * 96.0, device="cuda")) < 1e-2
    assert x.grad is not None and lin.weight.grad is not None
