"""Model families on CPU/gloo: every sharded model against the same model on one rank
(weights moved through the checkpoint module), and sharded checkpoints across meshes."""

import pytest
import torch

from dist_utils import assert_close, merge, run_distributed, singleton_mesh, split


def _grads_full(model):
    """Global gradients, assembled the same way as the global parameters."""
    from jigsaw_b200 import checkpoint

    layout = checkpoint.parameter_layout(model)
    out = {}
    for name, p in model.named_parameters():
        g = p.grad
        for dim, group in layout[name]:
            g = checkpoint.gather_dim(g, group, dim)
        out[name] = g
    return out


def _compare(dist_model, serial_model, y, y_ref_local, what, rtol=2e-4, atol=2e-5):
    from jigsaw_b200 import checkpoint

    assert_close(y, y_ref_local, f"{what}: output", rtol, atol)
    g_dist = _grads_full(dist_model)
    serial_grads = dict(serial_model.named_parameters())
    for name, g in g_dist.items():
        assert_close(g, serial_grads[name].grad, f"{what}: grad of {name}", 5 * rtol, 5 * atol)


def _worker_vit(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import ViT, ViTConfig

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    solo = singleton_mesh("row", "col")
    torch.manual_seed(1)
    x = torch.randn(2, 4, 16, 32)
    for seq, classes in (("ring", None), ("ulysses", 10)):
        cfg = ViTConfig(image_size=(16, 32), depth=2, num_classes=classes, sequence_parallel=seq, attn_backend="math")
        jb.launch.set_all_seeds(100 + mesh["model"].rank())
        model = ViT(mesh, "cpu", cfg)
        serial = ViT(solo, "cpu", cfg)
        # attention stores its qkv rows per channel rank: move it through the serial layout
        state = checkpoint.full_state_dict(model)
        checkpoint.load_full_state_dict(serial, state)
        xl = split(x, {1: mesh["col"], 3: mesh["row"]})
        y = model(xl)
        y_ref = serial(x)
        if classes is None:
            target = torch.zeros_like(x)
            loss = jb.modules.DistributedMSELoss(reduce_groups=(mesh["row"], mesh["col"]))(
                y, split(target, {1: mesh["col"], 3: mesh["row"]}))
            loss_ref = torch.nn.functional.mse_loss(y_ref, target)
            y_ref_local = split(y_ref.detach(), {1: mesh["col"], 3: mesh["row"]})
        else:
            labels = torch.tensor([3, 7])
            loss = jb.modules.DistributedCrossEntropyLoss(mesh["col"], (mesh["row"],))(y, labels)
            loss_ref = torch.nn.functional.cross_entropy(y_ref, labels)
            y_ref_local = split(y_ref.detach(), {1: mesh["col"]})
        assert_close(loss.detach(), loss_ref.detach(), f"vit {seq}: loss", 1e-4, 1e-6)
        loss.backward()
        loss_ref.backward()
        # compare gradients in the serial layout
        g = {n: p.grad for n, p in model.named_parameters()}
        for p in model.parameters():
            p.data, p.grad = p.grad, None
        g_full = checkpoint.full_state_dict(model)
        assert_close(y.detach(), y_ref_local, f"vit {seq}: output", 2e-4, 2e-5)
        for name, p in serial.named_parameters():
            assert_close(g_full[name], p.grad, f"vit {seq}: grad of {name}", 1e-3, 1e-5)


def test_vit_ring_and_ulysses_match_serial():
    run_distributed(_worker_vit, 4)


def _worker_swin(rank, world, axes):
    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import Swin, SwinConfig

    mesh = jb.make_process_mesh(axes)
    solo = singleton_mesh("sh", "sw", "col")
    for classes in (None, 6):
        cfg = SwinConfig(image_size=(32, 32), in_channels=2, patch=2, dims=(8, 16), heads=(2, 4), depths=(2, 2), window=4,
                         num_classes=classes)
        jb.launch.set_all_seeds(7 + mesh["col"].rank())
        model = Swin(mesh, "cpu", cfg)
        serial = Swin(solo, "cpu", cfg)
        checkpoint.load_full_state_dict(serial, checkpoint.full_state_dict(model))
        torch.manual_seed(3)
        x = torch.randn(2, 2, 32, 32)
        cuts = {1: mesh["col"], 2: mesh["sh"], 3: mesh["sw"]}
        y = model(split(x, cuts))
        y_ref = serial(x)
        assert_close(y.detach(), split(y_ref.detach(), cuts), f"swin {axes} classes={classes}: output", 2e-4, 2e-5)
        (y * split(torch.linspace(0, 1, y_ref.numel()).view_as(y_ref), cuts)).sum().backward()
        (y_ref * torch.linspace(0, 1, y_ref.numel()).view_as(y_ref)).sum().backward()
        for p in model.parameters():
            p.data, p.grad = p.grad, None
        g_full = checkpoint.full_state_dict(model)
        for name, p in serial.named_parameters():
            assert_close(g_full[name], p.grad, f"swin {axes}: grad of {name}", 2e-3, 2e-4)


@pytest.mark.parametrize("axes", [{"sh": 2, "sw": 2, "col": 1}, {"sh": 2, "sw": 1, "col": 2}])
def test_swin_matches_serial(axes):
    run_distributed(_worker_swin, 4, axes)


def _worker_unet(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import UNet3d, UNet3dConfig

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    solo = singleton_mesh("sh", "sw", "col")
    cfg = UNet3dConfig(widths=(8, 16), norm_groups=4)
    jb.launch.set_all_seeds(11)
    model, serial = UNet3d(mesh, "cpu", cfg), UNet3d(solo, "cpu", cfg)
    checkpoint.load_full_state_dict(serial, checkpoint.full_state_dict(model))
    torch.manual_seed(5)
    x = torch.randn(1, 1, 8, 16, 16)
    t = (torch.rand(1, 1, 8, 16, 16) > 0.5).float()
    cuts = {3: mesh["sh"], 4: mesh["sw"]}
    y = model(split(x, cuts))
    y_ref = serial(x)
    loss = jb.modules.DistributedBCEWithLogitsLoss(reduce_groups=(mesh["sh"], mesh["sw"]))(y, split(t, cuts))
    loss_ref = torch.nn.functional.binary_cross_entropy_with_logits(y_ref, t)
    assert_close(y.detach(), split(y_ref.detach(), cuts), "unet3d: output", 2e-4, 2e-5)
    assert_close(loss.detach(), loss_ref.detach(), "unet3d: loss", 1e-5, 1e-6)
    loss.backward()
    loss_ref.backward()
    for (n, p), (_, q) in zip(model.named_parameters(), serial.named_parameters()):
        assert_close(p.grad, q.grad, f"unet3d: grad of {n}", 2e-3, 1e-5)


def test_unet3d_matches_serial():
    run_distributed(_worker_unet, 4)


def _worker_checkpoint(rank, world, tmp):
    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import ViT, ViTConfig

    cfg = ViTConfig(image_size=(16, 32), depth=1, attn_backend="math")
    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    jb.launch.set_all_seeds(40 + rank)
    model = ViT(mesh, "cpu", cfg)
    torch.manual_seed(0)
    x = torch.randn(1, 4, 16, 32)
    y = merge(model(split(x, {1: mesh["col"], 3: mesh["row"]})).detach(), {1: mesh["col"], 3: mesh["row"]})
    checkpoint.save_sharded(model, mesh, tmp, extra={"step": 12})
    import os

    assert sorted(f for f in os.listdir(tmp) if f.endswith(".pt")) == [f"shard-col{c}-row{r}.pt" for c in (0, 1) for r in (0, 1)]
    for axes in ({"row": 2, "col": 2}, {"row": 4, "col": 1}, {"row": 1, "col": 4}, {"dp": 2, "row": 1, "col": 2}):
        kw = {"model_parallel_axes": ("row", "col")} if "dp" in axes else {}
        mesh2 = jb.make_process_mesh(axes, **kw)
        other = ViT(mesh2, "cpu", cfg)
        extra = checkpoint.load_sharded(other, mesh2, tmp)
        assert extra == {"step": 12}
        cuts = {1: mesh2["col"], 3: mesh2["row"]}
        y2 = merge(other(split(x, cuts)).detach(), cuts)
        assert_close(y2, y, f"checkpoint read back on {axes}", 2e-4, 2e-5)


def test_sharded_checkpoint_across_meshes(tmp_path):
    run_distributed(_worker_checkpoint, 4, str(tmp_path))


def _worker_checkpoint_plain_dict(rank, world, tmp):
    """A plain ``{name: group}`` mapping that also carries the flattened model group (the form the
    reference's ``process_mesh_dict`` has) names the same shards as the mesh object."""
    import os

    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import ViT, ViTConfig

    cfg = ViTConfig(image_size=(16, 32), depth=1, attn_backend="math")
    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    jb.launch.set_all_seeds(40 + rank)
    model = ViT(mesh, "cpu", cfg)
    plain = {"model": mesh["model"], "row": mesh["row"], "col": mesh["col"]}
    assert list(checkpoint._mesh_groups(plain)) == ["row", "col"]
    checkpoint.save_sharded(model, plain, tmp)
    assert sorted(f for f in os.listdir(tmp) if f.endswith(".pt")) == [f"shard-col{c}-row{r}.pt" for c in (0, 1) for r in (0, 1)]
    other = ViT(mesh, "cpu", cfg)
    checkpoint.load_sharded(other, plain, tmp)
    for (k, a), b in zip(model.state_dict().items(), other.state_dict().values()):
        assert_close(b, a, f"plain-dict checkpoint: {k}", 0, 0)


def test_sharded_checkpoint_with_a_plain_group_dict(tmp_path):
    run_distributed(_worker_checkpoint_plain_dict, 4, str(tmp_path))


def _worker_reshard_hops(rank, world):
    """The layers of a ViT (patch convolution, layer norms, attention, block linears) carried
    2x2 -> 1x4 -> 4x1 -> 2x2 with ``reshard_parameters``: after every hop the gathered state equals the
    original, and back on the first mesh the model computes what it computed before.  (On the meshes in
    between only the layers are valid: the model object keeps its own mesh-dependent buffers.)"""
    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import ViT, ViTConfig

    meshes = [jb.make_process_mesh({"row": 2, "col": 2}), jb.make_process_mesh({"row": 1, "col": 4}),
              jb.make_process_mesh({"row": 4, "col": 1})]
    cfg = ViTConfig(image_size=(16, 32), depth=1, heads=4, num_classes=None, sequence_parallel="ulysses", attn_backend="math")
    jb.launch.set_all_seeds(7 + meshes[0]["model"].rank())
    model = ViT(meshes[0], "cpu", cfg)
    torch.manual_seed(3)
    x = torch.randn(2, 4, 16, 32)
    xl = split(x, {1: meshes[0]["col"], 3: meshes[0]["row"]})
    with torch.no_grad():
        y0 = model(xl)
    state0 = {k: v.clone() for k, v in checkpoint.full_state_dict(model).items()}
    hops = [(0, 1), (1, 2), (2, 0)]
    for a, b in hops:
        for layer in model.modules():
            if hasattr(layer, "reshard_parameters"):
                layer.reshard_parameters(meshes[a], meshes[b])
        state = checkpoint.full_state_dict(model)
        assert state.keys() == state0.keys()
        for k in state0:
            assert_close(state[k], state0[k], f"hop {a}->{b}: {k}", 0, 0)
    with torch.no_grad():
        assert_close(model(xl), y0, "output after the round trip", 0, 1e-6)


def test_reshard_multi_hop_round_trip():
    run_distributed(_worker_reshard_hops, 4)


def _worker_resume(rank, world, tmp, which):
    """Two steps on a 2 x 2 mesh, checkpoint with the optimizer, two more steps on a 1 x 4 mesh from the
    checkpoint: the result equals four uninterrupted steps."""
    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import ViT, ViTConfig
    from jigsaw_b200.optim import FusedAdam

    cfg = ViTConfig(image_size=(16, 32), depth=1, heads=4, attn_backend="math")
    make_opt = (lambda ps: FusedAdam(ps, lr=1e-2)) if which == "fused" else (lambda ps: torch.optim.Adam(ps, lr=1e-2))
    torch.manual_seed(0)
    xs = [torch.randn(2, 4, 16, 32) for _ in range(4)]

    def train(model, opt, mesh, batches):
        cuts = {1: mesh["col"], 3: mesh["row"]}
        loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["row"], mesh["col"]))
        for x in batches:
            loss = loss_fn(model(split(x, cuts)), split(torch.zeros_like(x), cuts))
            opt.zero_grad()
            loss.backward()
            opt.step()

    mesh_a = jb.make_process_mesh({"row": 2, "col": 2})
    mesh_b = jb.make_process_mesh({"row": 1, "col": 4})
    jb.launch.set_all_seeds(11 + mesh_a["model"].rank())
    straight = ViT(mesh_a, "cpu", cfg)
    start = checkpoint.full_state_dict(straight)
    opt = make_opt(straight.parameters())
    train(straight, opt, mesh_a, xs)
    want = checkpoint.full_state_dict(straight)

    first = ViT(mesh_a, "cpu", cfg)
    checkpoint.load_full_state_dict(first, start)
    opt1 = make_opt(first.parameters())
    train(first, opt1, mesh_a, xs[:2])
    checkpoint.save_sharded(first, mesh_a, tmp, extra={"step": 2}, optimizer=opt1)
    second = ViT(mesh_b, "cpu", cfg)
    opt2 = make_opt(second.parameters())
    for g in opt2.param_groups:
        g["lr"] = 123.0                                    # must be replaced by the saved value
    assert checkpoint.load_sharded(second, mesh_b, tmp, optimizer=opt2) == {"step": 2}
    assert opt2.param_groups[0]["lr"] == 1e-2
    train(second, opt2, mesh_b, xs[2:])
    got = checkpoint.full_state_dict(second)
    for k in want:
        assert_close(got[k], want[k], f"{which}: {k} after resuming on another mesh", 1e-4, 1e-6)


@pytest.mark.parametrize("which", ["fused", "torch"])
def test_resume_with_optimizer_on_another_mesh(tmp_path, which):
    run_distributed(_worker_resume, 4, str(tmp_path), which)


def _worker_recompute(rank, world):
    """Activation checkpointing of the transformer blocks (ring and Ulysses attention inside) leaves the
    loss and every gradient unchanged."""
    import dataclasses

    import jigsaw_b200 as jb
    from jigsaw_b200.models import ViT, ViTConfig

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    torch.manual_seed(2)
    x = torch.randn(2, 4, 16, 32)
    cuts = {1: mesh["col"], 3: mesh["row"]}
    for seq in ("ring", "ulysses"):
        cfg = ViTConfig(image_size=(16, 32), depth=2, heads=4, sequence_parallel=seq, attn_backend="math")
        jb.launch.set_all_seeds(5 + mesh["model"].rank())
        plain = ViT(mesh, "cpu", cfg)
        saving = ViT(mesh, "cpu", dataclasses.replace(cfg, recompute_blocks=True))
        saving.load_state_dict(plain.state_dict())
        loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["row"], mesh["col"]))
        outs = []
        for model in (plain, saving):
            loss = loss_fn(model(split(x, cuts)), split(torch.zeros_like(x), cuts))
            loss.backward()
            outs.append(loss.detach())
        assert_close(outs[1], outs[0], f"{seq}: loss with recomputation", 0, 1e-7)
        for (n, p), q in zip(plain.named_parameters(), saving.parameters()):
            assert_close(q.grad, p.grad, f"{seq}: gradient of {n} with recomputation", 1e-5, 1e-7)


def test_vit_block_recomputation_keeps_gradients():
    run_distributed(_worker_recompute, 4)


def _worker_recompute_swin(rank, world):
    """The same for the Swin layers (rolls, window attention, patch merging inside the recomputed part)."""
    import dataclasses

    import jigsaw_b200 as jb
    from jigsaw_b200.models import Swin, SwinConfig

    mesh = jb.make_process_mesh({"sh": 2, "sw": 1, "col": 2})
    cfg = SwinConfig(image_size=(32, 32), in_channels=2, patch=2, dims=(8, 16), heads=(2, 4), depths=(2, 2), window=4)
    jb.launch.set_all_seeds(7 + mesh["col"].rank())
    plain = Swin(mesh, "cpu", cfg)
    saving = Swin(mesh, "cpu", dataclasses.replace(cfg, recompute_blocks=True))
    saving.load_state_dict(plain.state_dict())
    torch.manual_seed(3)
    x = torch.randn(2, 2, 32, 32)
    cuts = {1: mesh["col"], 2: mesh["sh"], 3: mesh["sw"]}
    for model in (plain, saving):
        model(split(x, cuts)).square().sum().backward()
    for (n, p), q in zip(plain.named_parameters(), saving.parameters()):
        assert_close(q.grad, p.grad, f"swin: gradient of {n} with recomputation", 1e-5, 1e-7)


def test_swin_layer_recomputation_keeps_gradients():
    run_distributed(_worker_recompute_swin, 4)


def _worker_reshard_refused(rank, world):
    """A mesh that does not divide the layer is refused on every rank, and the layer is left as it was."""
    import jigsaw_b200 as jb

    a = jb.make_process_mesh({"row": 2, "col": 2})
    b = jb.make_process_mesh({"row": 1, "col": 4})
    layers = [jb.modules.DistributedLinear(6, 6, "cpu", a["model"], a["row"], a["col"]),
              jb.modules.DistributedLayerNorm(6, a["model"].rank(), "cpu", a["row"], a["col"])]
    x = split(torch.randn(4, 6), {0: a["row"], 1: a["col"]})
    img = split(torch.randn(1, 4, 4, 8), {1: a["col"], 3: a["row"]})
    vol = split(torch.randn(1, 12, 4, 8), {1: a["col"], 3: a["row"]})
    inputs = [x, x, img, vol]
    layers += [jb.modules.DistributedConv2d(4, 6, 3, "cpu", a["row"], a["col"], padding=1),
               jb.modules.DistributedGroupNorm(2, 12, "cpu", channel_group=a["col"], spatial_group=a["row"])]
    for layer, x in zip(layers, inputs):
        before = [p.detach().clone() for p in layer.parameters()]
        y = layer(x).detach()
        with pytest.raises(ValueError):
            layer.reshard_parameters(a, b)
        for p, q in zip(layer.parameters(), before):
            assert_close(p.detach(), q, "parameters after a refused reshard", 0, 0)
        assert_close(layer(x).detach(), y, "forward after a refused reshard", 0, 0)


def test_reshard_onto_a_mesh_that_does_not_divide_is_refused():
    run_distributed(_worker_reshard_refused, 4)


def _worker_recompute_unet(rank, world):
    """Stage recomputation in the 3-D encoder (halo convolutions and tile-wide group norm inside the recomputed
    part) leaves the gradients unchanged."""
    import dataclasses

    import jigsaw_b200 as jb
    from jigsaw_b200.models import UNet3d, UNet3dConfig

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    cfg = UNet3dConfig(widths=(8, 16), norm_groups=4)
    jb.launch.set_all_seeds(11)
    plain = UNet3d(mesh, "cpu", cfg)
    saving = UNet3d(mesh, "cpu", dataclasses.replace(cfg, recompute_stages=True))
    saving.load_state_dict(plain.state_dict())
    torch.manual_seed(5)
    x = split(torch.randn(1, 1, 8, 16, 16), {3: mesh["sh"], 4: mesh["sw"]})
    for model in (plain, saving):
        model(x).square().sum().backward()
    for (n, p), q in zip(plain.named_parameters(), saving.parameters()):
        assert_close(q.grad, p.grad, f"unet3d: gradient of {n} with recomputation", 1e-5, 1e-7)


def test_unet3d_stage_recomputation_keeps_gradients():
    run_distributed(_worker_recompute_unet, 4)
