"""tcgen05 GEMM kernel and the fused linear layer on one GPU against fp32 PyTorch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 384, 192), (1000, 520, 328), (4096, 1024, 512)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from jigsaw_b200.ops import linear_fused, symm

    if M % 8 or N % 8 or K % 8:
        pytest.skip("leading dimensions must be multiples of 8")
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    A = torch.randn(M, K, device=dev).to(torch.bfloat16)
    B = torch.randn(N, K, device=dev).to(torch.bfloat16)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    out = linear_fused.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    symm.arena(dev).check_status()
    assert _rel(out, ref) < 2e-3
    bias = torch.randn(N, device=dev)
    out = linear_fused.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, gelu=True)
    assert _rel(out, torch.nn.functional.gelu(ref + bias)) < 2e-2


def test_fused_linear_forward_backward():
    from jigsaw_b200.ops import _lib, linear_fused

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    x = torch.randn(4, 200, 256, device=dev, requires_grad=True)
    lin = torch.nn.Linear(256, 384, device=dev)
    g = torch.randn(4, 200, 384, device=dev)
    before = _lib.LAUNCHES
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = linear_fused.maybe_fused_linear(x, lin.weight, lin.bias)
    assert y is not None and y.dtype == torch.bfloat16
    y.backward(g.to(torch.bfloat16))
    assert _lib.LAUNCHES == before + 3
    xr = x.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, lin.weight.detach(), lin.bias.detach())
    wr = lin.weight.detach().clone().requires_grad_(True)
    br = lin.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g)
    assert _rel(y, yr) < 2e-2
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(lin.weight.grad, wr.grad) < 2e-2
    assert _rel(lin.bias.grad, br.grad) < 2e-2
    assert linear_fused.maybe_fused_linear(x, lin.weight, lin.bias) is None      # fp32 outside autocast: torch path
