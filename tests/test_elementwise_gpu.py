"""Kernels on one GPU against plain PyTorch fp32: chunk merge, squared-error loss (strided / bf16),
multi-tensor Adam and gradient norm, cross-entropy, and the tcgen05 attention kernels (plain and over
several parts of the sequence)."""

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


@pytest.mark.parametrize("kind", ["l1", "smooth_l1", "bce", "bce_logits"])
@pytest.mark.parametrize("shape,channels_last,dtype", [((2, 3, 40, 50), True, torch.bfloat16), ((3, 1000), False, torch.float32)])
def test_pair_loss_kernels(kind, shape, channels_last, dtype):
    """L1, smooth L1 and the two binary cross-entropies on the fused element-wise loss kernels (one launch
    per direction) against torch.nn.functional on fp32 copies of the same values."""
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib

    F, JF = torch.nn.functional, jb.modules.functional
    ours, theirs, kw = {"l1": (JF.distributed_l1_loss, F.l1_loss, {}),
                        "smooth_l1": (JF.distributed_smooth_l1_loss, F.smooth_l1_loss, {"beta": 0.7}),
                        "bce": (JF.distributed_binary_cross_entropy, F.binary_cross_entropy, {}),
                        "bce_logits": (JF.distributed_binary_cross_entropy_with_logits, F.binary_cross_entropy_with_logits, {})}[kind]
    torch.manual_seed(4)
    a = torch.rand(*shape, device=DEV) * 0.98 + 0.01 if kind == "bce" else torch.randn(*shape, device=DEV) * 2
    if channels_last:
        a = a.permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)
    a = a.to(dtype).requires_grad_(True)
    b = torch.rand(*shape, device=DEV) if kind.startswith("bce") else torch.randn(*shape, device=DEV)
    before = _lib.LAUNCHES
    with _lib.strict_fused():
        loss = ours(a, b, **kw)
    loss.backward()
    assert _lib.LAUNCHES == before + 2
    ar = a.detach().float().requires_grad_(True)
    ref = theirs(ar, b, **kw)
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


def _attention_reference(q, k, v, g, scale):
    """fp32 attention of the same bf16 inputs with autograd: (out, lse, dq, dk, dv)."""
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    t = scale * (qf @ kf.transpose(-1, -2))
    out = torch.softmax(t, dim=-1) @ vf
    out.backward(g.float())
    return out.detach(), torch.logsumexp(t.detach(), dim=-1), qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("shape", [(2, 3, 128, 128), (1, 2, 300, 520), (1, 3, 256, 384), (2, 4, 1024, 2048)])
def test_flash_attention_forward_backward(shape):
    """tcgen05 attention (head dimension 64) against fp32 attention of the same bf16 inputs: output,
    log-sum-exp and the three gradients; sequence lengths that do and do not fill the 128-row tiles."""
    from jigsaw_b200.ops import attention_fused, symm

    b, h, sq, sk = shape
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    q = torch.randn(b, h, sq, 64, device=dev).bfloat16()
    k = torch.randn(b, h, sk, 64, device=dev).bfloat16()
    v = torch.randn(b, h, sk, 64, device=dev).bfloat16()
    g = torch.randn(b, h, sq, 64, device=dev).bfloat16()
    scale = 0.125
    ref, ref_lse, rq, rk, rv = _attention_reference(q, k, v, g, scale)
    out, lse = attention_fused.flash_attention_forward(q, k, v, scale)
    torch.cuda.synchronize()
    symm.arena(dev).check_status()
    assert float((lse - ref_lse).abs().max()) < 2e-2
    assert float((out.float() - ref).abs().max()) < 2e-2 * float(ref.abs().max())
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    attention_fused.FlashAttention.apply(qg, kg, vg, scale).backward(g)
    torch.cuda.synchronize()
    symm.arena(dev).check_status()
    for name, mine, ref_g in (("dq", qg.grad, rq), ("dk", kg.grad, rk), ("dv", vg.grad, rv)):
        assert float((mine.float() - ref_g).abs().max()) < 2e-2 * float(ref_g.abs().max()), name


def test_flash_attention_growing_maximum():
    """Scores whose row maximum keeps growing along the keys (each block of 128 keys is scaled up), so that
    the lazily rescaled accumulator of the forward kernel is rescaled several times."""
    from jigsaw_b200.ops import attention_fused, symm

    dev = torch.device("cuda", 0)
    torch.manual_seed(6)
    q = torch.randn(1, 2, 256, 64, device=dev).bfloat16()
    k = torch.randn(1, 2, 1024, 64, device=dev)
    k = (k * torch.linspace(0.5, 6.0, 8, device=dev).repeat_interleave(128).view(1, 1, -1, 1)).bfloat16()
    v = torch.randn(1, 2, 1024, 64, device=dev).bfloat16()
    g = torch.randn(1, 2, 256, 64, device=dev).bfloat16()
    ref, ref_lse, *_ = _attention_reference(q, k, v, g, 0.125)
    out, lse = attention_fused.flash_attention_forward(q, k, v, 0.125)
    torch.cuda.synchronize()
    symm.arena(dev).check_status()
    assert float((lse - ref_lse).abs().max()) < 2e-2
    assert float((out.float() - ref).abs().max()) < 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("parts,s_part", [(2, 256), (4, 128), (3, 200)])
def test_flash_attention_over_parts_on_one_gpu(parts, s_part):
    """The multi-part entry points that carry ring attention, with every part in this GPU's memory: the keys
    and values (forward, dQ) and the queries, output gradients, log-sum-exp and D (dK / dV) are walked part by
    part, starting from the caller's own, and must give attention over the concatenated sequence."""
    import ctypes

    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", 0)
    torch.manual_seed(7)
    bh, scale = 6, 0.125
    S = parts * s_part
    q, k, v, g = (torch.randn(bh, S, 64, device=dev).bfloat16() for _ in range(4))
    ref, ref_lse, rq, rk, rv = _attention_reference(q, k, v, g, scale)
    L, ar = _lib.lib(), symm.arena(dev)
    P_ = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    cut = lambda t: [t[:, p * s_part:(p + 1) * s_part].contiguous() for p in range(parts)]  # noqa: E731
    qs, ks, vs, gs = cut(q), cut(k), cut(v), cut(g)

    def ptrs(ts):
        arr = (ctypes.c_void_p * 8)()
        for i, t in enumerate(ts):
            arr[i] = t.data_ptr()
        return arr

    outs, lses, deltas = [], [], []
    for me in range(parts):
        out = torch.empty(bh, s_part, 64, device=dev, dtype=torch.bfloat16)
        lse = torch.empty(bh, s_part, device=dev)
        rc = L.jb_flash_attn_fwd_parts(P_(qs[me]), ptrs(ks), ptrs(vs), None, 0, 0, None, parts, me, P_(out), P_(lse), bh, s_part,
                                       s_part, 64, s_part * 64, 64, s_part * 64, 64, s_part * 64, scale, P_(ar.status),
                                       _lib.stream_ptr())
        assert rc == 0
        delta = torch.empty(bh, s_part, device=dev)
        assert L.jb_flash_attn_delta(P_(out), P_(gs[me]), P_(delta), bh * s_part, _lib.stream_ptr()) == 0
        outs.append(out)
        lses.append(lse)
        deltas.append(delta)
    torch.cuda.synchronize()
    ar.check_status()
    out_all, lse_all = torch.cat(outs, dim=1), torch.cat(lses, dim=1)
    assert float((lse_all - ref_lse).abs().max()) < 2e-2
    assert float((out_all.float() - ref).abs().max()) < 2e-2 * float(ref.abs().max())
    dqs, dks, dvs = [], [], []
    for me in range(parts):
        dq, dk, dv = (torch.empty(bh, s_part, 64, device=dev, dtype=torch.bfloat16) for _ in range(3))
        rc = L.jb_flash_attn_bwd_parts(P_(qs[me]), P_(ks[me]), P_(vs[me]), P_(gs[me]), ptrs(qs), ptrs(gs), ptrs(lses), ptrs(deltas),
                                       ptrs(ks), ptrs(vs), None, 0, 0, None, parts, me, P_(dq), P_(dk), P_(dv), bh, s_part, scale,
                                       P_(ar.status), _lib.stream_ptr())
        assert rc == 0
        dqs.append(dq)
        dks.append(dk)
        dvs.append(dv)
    torch.cuda.synchronize()
    ar.check_status()
    for name, mine, ref_g in (("dq", torch.cat(dqs, 1), rq), ("dk", torch.cat(dks, 1), rk), ("dv", torch.cat(dvs, 1), rv)):
        assert float((mine.float() - ref_g).abs().max()) < 2e-2 * float(ref_g.abs().max()), name
