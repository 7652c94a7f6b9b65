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


@pytest.mark.parametrize("staged", [False, True])
@pytest.mark.parametrize("M,K,part_cols,b_mn", [(300, 256, 256, False), (9516, 128, 256, True), (520, 192, 64, False)])
def test_scatter_epilogue_into_local_slabs(M, K, part_cols, b_mn, staged):
    """The GEMM whose epilogue stores column part ``p`` of the product into slab ``p``; here both slabs
    are buffers of this GPU, so that the epilogue's addressing is checked without peers.  The staged
    form (tiles leave through shared memory as 128-byte row pieces) runs only when
    JIGSAW_STAGED_EPILOGUE=1 is set: it has not been measured on hardware yet."""
    import ctypes
    import os

    from jigsaw_b200.ops import _lib, symm

    if staged and os.environ.get("JIGSAW_STAGED_EPILOGUE", "0") != "1":
        pytest.skip("set JIGSAW_STAGED_EPILOGUE=1 to run the staged epilogue")
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    parts = 2
    N = parts * part_cols
    A = torch.randn(M, K, device=dev).bfloat16()
    B = torch.randn(N, K, device=dev).bfloat16()
    b = B.t().contiguous() if b_mn else B
    slabs = [torch.full((M, part_cols), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(parts)]
    c_part = (ctypes.c_void_p * 8)()
    for i, t in enumerate(slabs):
        c_part[i] = t.data_ptr()
    L = _lib.lib()
    ar = symm.arena(dev)
    fn = L.jb_gemm_bf16_scatter_staged if staged else L.jb_gemm_bf16_scatter
    rc = fn(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(b.data_ptr()), c_part, parts, part_cols, M, K, A.stride(0),
            b.stride(0), 0, 1 if b_mn else 0, _lib.sm_count(0), ctypes.c_void_p(ar.status.data_ptr()), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    ar.check_status()
    ref = A.float() @ B.float().t()
    for i, t in enumerate(slabs):
        assert not torch.isnan(t).any(), f"slab {i} has rows the epilogue did not write"
        assert _rel(t, ref[:, i * part_cols:(i + 1) * part_cols]) < 1e-2
