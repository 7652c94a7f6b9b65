"""Fused sm_100a convolution kernels against plain PyTorch fp32 references (1 GPU)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_chain(x, weights, biases):
    h = x
    for i, (w, b) in enumerate(zip(weights, biases)):
        h = torch.nn.functional.conv2d(h, w, b, padding=1)
        if i + 1 < len(weights):
            h = torch.nn.functional.gelu(h)
    return h


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12))


@pytest.mark.parametrize("shape", [(1, 24, 256), (2, 37, 200)])
def test_chain_forward_backward_matches_fp32(shape):
    from jigsaw_b200.ops import conv_fused, symm

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    NB, H, W = shape
    chans = [3, 64, 64, 64, 3]
    ws = [(torch.randn(chans[i + 1], chans[i], 3, 3, device=dev) * (2.0 / (9 * chans[i])) ** 0.5).requires_grad_(True)
          for i in range(4)]
    bs = [(torch.randn(chans[i + 1], device=dev) * 0.1).requires_grad_(True) for i in range(4)]
    x = torch.randn(NB, 3, H, W, device=dev)
    geom = conv_fused.geometry_for(x, None, None)
    kinds = conv_fused.chain_kinds([(chans[i], chans[i + 1]) for i in range(4)])
    assert kinds == ["thin_in", "mid", "mid", "thin_out"]
    out = conv_fused.conv_chain(x, geom, kinds, [True, True, True, False], ws, bs)
    gout = torch.randn_like(out)
    out.backward(gout)
    got = [p.grad.clone() for p in ws + bs]
    for p in ws + bs:
        p.grad = None
    # reference: same bf16-rounded operands, fp32 math
    ref = _ref_chain(x, ws, bs)
    ref.backward(gout.float())
    assert _rel(out, ref) < 3e-2
    for g, p in zip(got, ws + bs):
        assert _rel(g, p.grad) < 5e-2, (tuple(p.shape), _rel(g, p.grad))
    symm.arena(dev).check_status()


def test_single_mid_layer_input_gradient():
    from jigsaw_b200.ops import conv_fused, symm

    torch.manual_seed(1)
    dev = torch.device("cuda", 0)
    x = torch.randn(1, 64, 20, 130, device=dev, requires_grad=True)
    w = (torch.randn(64, 64, 3, 3, device=dev) * 0.05).requires_grad_(True)
    b = torch.randn(64, device=dev).requires_grad_(True)
    geom = conv_fused.geometry_for(x, None, None)
    out = conv_fused.conv_chain(x, geom, ["mid"], [False], [w], [b])
    gout = torch.randn_like(out)
    out.backward(gout)
    gx, gw, gb = x.grad.clone(), w.grad.clone(), b.grad.clone()
    x.grad = w.grad = b.grad = None
    ref = torch.nn.functional.conv2d(x, w, b, padding=1)
    ref.backward(gout.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(gx, x.grad) < 2e-2 and _rel(gw, w.grad) < 2e-2 and _rel(gb, b.grad) < 2e-2
    symm.arena(dev).check_status()


def test_domain_cnn_module_uses_fused_chain_and_trains():
    import jigsaw_b200 as jb
    from jigsaw_b200.models import DomainCNN
    import torch.distributed as dist

    dev = torch.device("cuda", 0)
    if not dist.is_initialized():
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1, device_id=dev)
    mesh = jb.make_process_mesh({"sh": 1, "sw": 1, "col": 1})
    torch.manual_seed(0)
    model = DomainCNN(mesh, dev, depth=4)
    x = torch.randn(1, 3, 64, 128, device=dev)
    y = torch.randn(1, 3, 64, 128, device=dev)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(x)
    assert out.dtype == torch.bfloat16 and out.shape == (1, 3, 64, 128)
    loss = loss_fn(out.float(), y)
    loss.backward()
    model_ref = DomainCNN(mesh, dev, depth=4, fuse=False)
    model_ref.load_state_dict(model.state_dict())
    loss_ref = loss_fn(model_ref(x), y)
    loss_ref.backward()
    assert abs(float(loss) - float(loss_ref)) < 2e-2 * abs(float(loss_ref))
    for p, q in zip(model.parameters(), model_ref.parameters()):
        assert _rel(p.grad, q.grad) < 6e-2
    dist.destroy_process_group()
