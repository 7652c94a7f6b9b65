"""Fused LayerNorm kernels on one GPU against a plain PyTorch fp32 reference of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,n,dtype,affine", [
    ((37,), 64, torch.float32, True),
    ((3, 50), 512, torch.bfloat16, True),
    ((2000,), 1024, torch.bfloat16, True),
    ((129,), 260, torch.float32, False),
])
def test_layer_norm_matches_torch(rows, n, dtype, affine):
    from jigsaw_b200.ops import norm_fused, symm

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    x = (torch.randn(*rows, n, device=dev) * 2 + 0.5).to(dtype).requires_grad_(True)
    w = (torch.rand(n, device=dev) + 0.5).requires_grad_(True) if affine else None
    b = torch.randn(n, device=dev).requires_grad_(True) if affine else None
    g = torch.randn(*rows, n, device=dev).to(dtype)
    y = norm_fused.maybe_fused_layer_norm(x, w, b, None, 1e-5)
    assert y is not None and y.dtype == dtype
    y.backward(g)
    symm.arena(dev).check_status()
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True) if affine else None
    br = b.detach().clone().requires_grad_(True) if affine else None
    yr = torch.nn.functional.layer_norm(xr, (n,), wr, br, 1e-5)
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    torch.testing.assert_close(y.float(), yr, rtol=tol, atol=tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=tol, atol=tol * max(1.0, float(xr.grad.abs().max())))
    if affine:
        scale = float(wr.grad.abs().max())
        torch.testing.assert_close(w.grad, wr.grad, rtol=1e-4, atol=1e-4 * scale)
        torch.testing.assert_close(b.grad, br.grad, rtol=1e-4, atol=1e-4 * float(br.grad.abs().max()))


def test_layer_norm_module_uses_the_kernel_and_autocast_gives_fp32():
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib

    dev = torch.device("cuda", 0)
    ln = jb.modules.DistributedLayerNorm(256, None, dev, None, None)
    x = torch.randn(4, 33, 256, device=dev, dtype=torch.bfloat16)
    before = _lib.LAUNCHES
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = ln(x)
    assert _lib.LAUNCHES == before + 1 and y.dtype == torch.float32
    torch.testing.assert_close(y, torch.nn.functional.layer_norm(x.float(), (256,), ln.weight, ln.bias), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("shape,groups,dtype", [((2, 32, 16, 12, 8), 8, torch.float32), ((1, 16, 40, 36), 4, torch.bfloat16),
                                                ((3, 8, 100), 2, torch.float32)])
def test_group_norm_matches_torch(shape, groups, dtype):
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    gn = jb.modules.DistributedGroupNorm(groups, shape[1], dev)
    with torch.no_grad():
        gn.weight.uniform_(0.5, 1.5)
        gn.bias.normal_()
    x = (torch.randn(*shape, device=dev) * 2 + 1).to(dtype).requires_grad_(True)
    g = torch.randn(*shape, device=dev).to(dtype)
    for _ in range(2):                      # twice: the barrier counters must be left at zero
        x.grad = None
        gn.zero_grad()
        before = _lib.LAUNCHES
        y = gn(x)
        y.backward(g)
        assert _lib.LAUNCHES == before + 2
    symm.arena(dev).check_status()
    xr = x.detach().float().requires_grad_(True)
    wr, br = gn.weight.detach().clone().requires_grad_(True), gn.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.group_norm(xr, groups, wr, br, 1e-5)
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    torch.testing.assert_close(y.float(), yr, rtol=tol, atol=tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=tol, atol=tol * max(1.0, float(xr.grad.abs().max())))
    torch.testing.assert_close(gn.weight.grad, wr.grad, rtol=1e-3, atol=1e-3 * float(wr.grad.abs().max()))
    torch.testing.assert_close(gn.bias.grad, br.grad, rtol=1e-3, atol=1e-3 * float(br.grad.abs().max()))
