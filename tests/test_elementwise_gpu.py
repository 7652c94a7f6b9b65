"""Memory-bound helper kernels on one GPU against plain PyTorch fp32: chunk merge, squared-error
loss (strided / bf16), multi-tensor Adam and gradient norm."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_merge_chunks():
    from jigsaw_b200.modules.attention._cores import merge_chunks
    from jigsaw_b200.ops import _lib

    torch.manual_seed(0)
    out = torch.randn(2, 3, 50, 64, device=DEV)
    lse = torch.randn(2, 3, 50, device=DEV)
    lse[0, 0, :5] = float("-inf")                    # nothing merged yet for these rows
    for dtype in (torch.bfloat16, torch.float32):
        o2 = torch.randn(2, 3, 50, 64, device=DEV).to(dtype)
        l2 = torch.randn(2, 3, 50, device=DEV)
        w = torch.sigmoid(l2 - lse).unsqueeze(-1)
        ref_o, ref_l = out + w * (o2.float() - out), torch.logaddexp(lse, l2)
        before = _lib.LAUNCHES
        got_o, got_l = merge_chunks(out.clone(), lse.clone(), o2, l2)
        assert _lib.LAUNCHES == before + 1
        torch.testing.assert_close(got_o, ref_o, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(got_l, ref_l, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("shape,channels_last,dtype", [((2, 3, 40, 50), True, torch.bfloat16), ((2, 3, 40, 50), False, torch.float32),
                                                       ((5, 1000), False, torch.bfloat16), ((7,), False, torch.float32)])
def test_mse_loss_kernel(shape, channels_last, dtype):
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib

    torch.manual_seed(1)
    a = torch.randn(*shape, device=DEV)
    if channels_last:
        a = a.permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)       # NCHW view of NHWC memory
    a = a.to(dtype).requires_grad_(True)
    b = torch.randn(*shape, device=DEV)
    before = _lib.LAUNCHES
    loss = jb.modules.DistributedMSELoss(reduce_groups=None)(a, b)
    loss.backward()
    assert _lib.LAUNCHES == before + 2
    ar = a.detach().float().requires_grad_(True)
    ref = torch.nn.functional.mse_loss(ar, b)
    ref.backward()
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(loss.float(), ref, rtol=tol, atol=tol)
    assert a.grad.stride() == a.stride() and a.grad.dtype == dtype
    torch.testing.assert_close(a.grad.float(), ar.grad, rtol=tol, atol=tol * float(ar.grad.abs().max()))


@pytest.mark.parametrize("adamw", [False, True])
def test_fused_adam_matches_torch(adamw):
    from jigsaw_b200.optim import FusedAdam, fused_grad_norm

    torch.manual_seed(2)
    shapes = [(64, 64, 3, 3), (64,), (5000,), (3, 7)] * 14          # 56 tensors: two launches
    ours = [torch.randn(*s, device=DEV, requires_grad=True) for s in shapes]
    theirs = [p.detach().clone().requires_grad_(True) for p in ours]
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt_a = FusedAdam(ours, decoupled_weight_decay=adamw, **kw)
    opt_b = (torch.optim.AdamW if adamw else torch.optim.Adam)(theirs, **kw)
    for _ in range(4):
        for p, q in zip(ours, theirs):
            g = torch.randn_like(p)
            p.grad, q.grad = g.clone(), g.clone()
        norm = fused_grad_norm([p.grad for p in ours])
        ref_norm = torch.sqrt(sum(q.grad.pow(2).sum() for q in theirs))
        torch.testing.assert_close(norm, ref_norm, rtol=1e-5, atol=1e-5)
        opt_a.step()
        opt_b.step()
    for p, q in zip(ours, theirs):
        torch.testing.assert_close(p, q, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("shape,dtype", [((8, 1000), torch.float32), ((2, 19, 30, 40), torch.bfloat16), ((300, 16), torch.float32)])
@pytest.mark.parametrize("reduction", ["mean", "none"])
def test_cross_entropy_kernel(shape, dtype, reduction):
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib

    torch.manual_seed(3)
    x = (torch.randn(*shape, device=DEV) * 3).to(dtype).requires_grad_(True)
    tshape = (shape[0], *shape[2:])
    t = torch.randint(0, shape[1], tshape, device=DEV)
    t.view(-1)[::7] = -100
    before = _lib.LAUNCHES
    loss = jb.modules.functional.distributed_cross_entropy(x, t, reduction=reduction)
    (loss.sum() * 1.5).backward()
    assert _lib.LAUNCHES == before + 2
    xr = x.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xr, t, reduction=reduction)
    (ref.sum() * 1.5).backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(loss.float(), ref, rtol=tol, atol=tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=tol, atol=tol * max(float(xr.grad.abs().max()), 1e-3))


@pytest.mark.parametrize("shape", [(2, 3, 128, 128), (1, 2, 300, 520), (2, 4, 1024, 2048)])
def test_flash_attention_forward_backward(shape):
    """tcgen05 attention (head dimension 64) against fp32 attention of the same bf16 inputs: output,
    log-sum-exp and the three gradients.  The kernel has not run on hardware yet, so the test runs only when
    JIGSAW_FLASH_ATTENTION=1 is set."""
    import os

    if os.environ.get("JIGSAW_FLASH_ATTENTION", "0") != "1":
        pytest.skip("set JIGSAW_FLASH_ATTENTION=1 to run the tcgen05 attention forward")
    from jigsaw_b200.ops import attention_fused, symm

    b, h, sq, sk = shape
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    q = torch.randn(b, h, sq, 64, device=dev).bfloat16()
    k = torch.randn(b, h, sk, 64, device=dev).bfloat16()
    v = torch.randn(b, h, sk, 64, device=dev).bfloat16()
    scale = 0.125
    out, lse = attention_fused.flash_attention_forward(q, k, v, scale)
    torch.cuda.synchronize()
    symm.arena(dev).check_status()
    t = scale * (q.float() @ k.float().transpose(-1, -2))
    ref_lse = torch.logsumexp(t, dim=-1)
    ref = torch.softmax(t, dim=-1) @ v.float()
    assert float((lse - ref_lse).abs().max()) < 2e-2
    assert float((out.float() - ref).abs().max()) < 3e-2 * float(ref.abs().max())
    # backward kernels against autograd of the fp32 formulation
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    g = torch.randn(b, h, sq, 64, device=dev).bfloat16()
    (torch.softmax(scale * (qf @ kf.transpose(-1, -2)), dim=-1) @ vf).backward(g.float())
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    attention_fused.FlashAttention.apply(qg, kg, vg, scale).backward(g)
    torch.cuda.synchronize()
    symm.arena(dev).check_status()
    for name, mine, ref_g in (("dq", qg.grad, qf.grad), ("dk", kg.grad, kf.grad), ("dv", vg.grad, vf.grad)):
        assert float((mine.float() - ref_g).abs().max()) < 4e-2 * float(ref_g.abs().max()), name
