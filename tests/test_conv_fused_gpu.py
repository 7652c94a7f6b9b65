"""Fused sm_100a convolution kernels against plain PyTorch fp32 references (1 GPU)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _round(t):
    """bf16 rounding that gradients pass through unchanged (what the kernels do to every tensor they store)."""
    return t + (t.to(torch.bfloat16).float() - t).detach()


def _ref_chain(x, weights, biases):
    """fp32 math on the operands the kernels see: bf16-rounded input, weights and inter-layer activations."""
    h = _round(x)
    for i, (w, b) in enumerate(zip(weights, biases)):
        h = torch.nn.functional.conv2d(h, _round(w), b, padding=1)
        if i + 1 < len(weights):
            h = _round(torch.nn.functional.gelu(h))
    return h


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12))


@pytest.mark.parametrize("shape", [(1, 24, 256), (2, 37, 200), (1, 20, 131)])
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
    assert _rel(out, ref) < 1e-2
    for g, p in zip(got, ws + bs):
        assert _rel(g, p.grad) < 3e-2, (tuple(p.shape), _rel(g, p.grad))
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
    ref = torch.nn.functional.conv2d(_round(x), _round(w), b, padding=1)
    ref.backward(gout.float())
    assert _rel(out, ref) < 1e-2
    assert _rel(gx, x.grad) < 1e-2 and _rel(gw, w.grad) < 1e-2 and _rel(gb, b.grad) < 1e-2
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


def _one_rank_mesh(port):
    import torch.distributed as dist

    import jigsaw_b200 as jb

    dev = torch.device("cuda", 0)
    if not dist.is_initialized():
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1, device_id=dev)
    return jb.make_process_mesh({"sh": 1, "sw": 1, "col": 1}), dev


def test_layers_in_a_sequential_run_as_one_fused_chain():
    """``nn.Sequential(DistributedConv2d, nn.GELU, ...)`` (what the reference's users write) must run exactly
    the fused chain of ``DomainCNN``: the same kernels, the same number of launches, bit-identical output and
    gradients, with no layer declined (strict dispatch)."""
    import torch.distributed as dist

    import jigsaw_b200 as jb
    from jigsaw_b200.models import DomainCNN
    from jigsaw_b200.ops import _lib
    from jigsaw_b200.ops.lazy_chain import LazyConvChain

    mesh, dev = _one_rank_mesh(29534)
    torch.manual_seed(0)
    model = DomainCNN(mesh, dev, depth=4)
    layers = []
    for i, conv in enumerate(model.convs):
        twin = jb.modules.DistributedConv2d(conv.in_channels, conv.out_channels, 3, dev, (mesh["sh"], mesh["sw"]), mesh["col"], padding=1)
        twin.load_state_dict(conv.state_dict())
        layers.append(twin)
        if i + 1 < len(model.convs):
            layers.append(torch.nn.GELU())
    seq = torch.nn.Sequential(*layers)
    x = torch.randn(2, 3, 48, 160, device=dev)
    y = torch.randn(2, 3, 48, 160, device=dev)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    results = []
    for net in (model, seq):
        before = _lib.LAUNCHES
        _lib.dispatch_counts(reset=True)
        with _lib.strict_fused(), torch.autocast("cuda", dtype=torch.bfloat16):
            out = net(x)
            if net is seq:
                assert isinstance(out, LazyConvChain) and out.pending and len(out.layers) == 4
            loss = loss_fn(out, y)
        loss.backward()
        results.append((loss.detach().clone(), [p.grad.clone() for p in net.parameters()], _lib.LAUNCHES - before))
    counts = _lib.dispatch_counts()
    assert counts["conv2d"] == {"fused": 4, "fallback": 0}
    (l0, g0, n0), (l1, g1, n1) = results
    assert n0 == n1 and torch.equal(l0, l1)
    for a, b in zip(g0, g1):
        assert torch.equal(a, b)
    dist.destroy_process_group()


def test_converted_torch_cnn_takes_the_fused_path():
    """A plain torch CNN passed through ``convert_to_jigsaw`` runs on the fused kernels (strict dispatch) and
    matches the torch model in fp32."""
    import torch.distributed as dist

    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib

    mesh, dev = _one_rank_mesh(29535)
    torch.manual_seed(1)
    plain = torch.nn.Sequential(torch.nn.Conv2d(3, 64, 3, padding=1), torch.nn.GELU(), torch.nn.Conv2d(64, 64, 3, padding=1),
                                torch.nn.GELU(), torch.nn.Conv2d(64, 2, 3, padding=1)).to(dev)
    import copy

    dist_model = jb.convert.convert_to_jigsaw(copy.deepcopy(plain), mesh, dev, row_kw="sh", col_kw="col", model_kw="col",
                                              spatial_group=(mesh["sh"], mesh["sw"]))
    assert all(isinstance(m, (jb.modules.DistributedConv2d, torch.nn.GELU)) for m in dist_model)
    x = torch.randn(1, 3, 40, 136, device=dev)
    before = _lib.LAUNCHES
    with _lib.strict_fused(), torch.autocast("cuda", dtype=torch.bfloat16):
        out = dist_model(x).float()
    assert _lib.LAUNCHES - before == 4          # pack + three convolutions
    ref = _ref_chain(x, [m.weight for m in plain if isinstance(m, torch.nn.Conv2d)], [m.bias for m in plain if isinstance(m, torch.nn.Conv2d)])
    assert _rel(out, ref) < 1e-2
    dist.destroy_process_group()


@pytest.mark.parametrize("dims", [2, 3])
def test_patch_embedding_runs_on_the_own_gemm(dims):
    """A convolution whose kernel equals its stride (patch embedding) is one patch-gather copy and one tcgen05
    GEMM: output and all gradients against torch's convolution on bf16-rounded operands, strict dispatch."""
    import torch.distributed as dist

    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib

    mesh, dev = _one_rank_mesh(29536 + dims)
    torch.manual_seed(2)
    if dims == 2:
        layer = jb.modules.DistributedConv2d(4, 128, 16, dev, (mesh["sh"], mesh["sw"]), mesh["col"], stride=16)
        x = torch.randn(2, 4, 64, 96, device=dev, requires_grad=True)
        conv = torch.nn.functional.conv2d
    else:
        layer = jb.modules.DistributedConv3d(2, 64, 4, dev, (None, mesh["sh"], mesh["sw"]), mesh["col"], stride=4)
        x = torch.randn(1, 2, 8, 16, 24, device=dev, requires_grad=True)
        conv = torch.nn.functional.conv3d
    before = _lib.LAUNCHES
    with _lib.strict_fused(), torch.autocast("cuda", dtype=torch.bfloat16):
        y = layer(x)
    assert _lib.LAUNCHES == before + 1 and y.dtype == torch.bfloat16
    g = torch.randn_like(y)
    y.backward(g)
    got = (x.grad.clone(), layer.weight.grad.clone(), layer.bias.grad.clone())
    x.grad = None
    layer.zero_grad()
    ref = conv(_round(x), _round(layer.weight), layer.bias, stride=layer.stride)
    ref.backward(g.float())
    assert _rel(y, ref) < 1e-2
    for mine, theirs in zip(got, (x.grad, layer.weight.grad, layer.bias.grad)):
        assert _rel(mine, theirs) < 2e-2
    dist.destroy_process_group()
