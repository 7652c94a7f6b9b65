"""Multi-GPU tests of the fused halo-exchange convolution chain (peer stores over NVLink):
the fused chain on a tiled image must match the unfused torch + NCCL path of the same model,
which in turn is pinned against the undivided torch layers by the CPU tests."""

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed

pytestmark = pytest.mark.gpu


def _worker_chain(rank, world, mesh_shape):
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.models import DomainCNN
    from jigsaw_b200.ops import symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"sh": mesh_shape[0], "sw": mesh_shape[1], "col": 1})
    torch.manual_seed(0)
    fused = DomainCNN(mesh, dev, depth=4)
    plain = DomainCNN(mesh, dev, depth=4, fuse=False)
    plain.load_state_dict(fused.state_dict())
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(2, 3, 40, 136, generator=g).to(dev)
    y = torch.randn(2, 3, 40, 136, generator=g).to(dev)
    for step in range(2):      # twice: buffers, flag slots and epochs are recycled
        for m in (fused, plain):
            m.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out_f = fused(x)
        loss_f = loss_fn(out_f.float(), y)
        loss_f.backward()
        out_p = plain(x)                       # fp32 oracle through torch + NCCL halo exchange
        loss_p = loss_fn(out_p, y)
        loss_p.backward()
        symm.arena(dev).check_status()
        scale = float(out_p.abs().max())
        assert_close(out_f.float(), out_p, f"step {step}: output", 0.0, 3e-2 * scale)
        assert_close(loss_f, loss_p, f"step {step}: loss", 2e-2, 0.0)
        for (n, p), q in zip(fused.named_parameters(), plain.parameters()):
            gs = float(q.grad.abs().max())
            assert_close(p.grad, q.grad, f"step {step}: grad {n}", 0.0, 6e-2 * gs + 1e-7)
    jb.debug.assert_replica_consistency(fused, mesh)


@pytest.mark.multigpu(2)
def test_fused_chain_two_gpus_rows():
    run_distributed(_worker_chain, 2, (2, 1), backend="nccl", timeout=300)


@pytest.mark.multigpu(2)
def test_fused_chain_two_gpus_cols():
    run_distributed(_worker_chain, 2, (1, 2), backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_fused_chain_four_gpus_with_corners():
    run_distributed(_worker_chain, 4, (2, 2), backend="nccl", timeout=300)


def _delay_kernel(name: str, cycles: int) -> None:
    """Host-side injection of a lagging rank: every launch of the library function ``name`` is
    preceded, on the same stream, by a bounded device-side delay, so that this rank's kernels still
    read a buffer while the other rank is already far ahead."""
    from jigsaw_b200.ops import _lib

    L = _lib.lib()
    orig = getattr(L, name)

    def delayed(*args):
        torch.cuda._sleep(cycles)
        return orig(*args)

    setattr(L, name, delayed)


def _gathered_conv(x_local, layer, cuts, dev):
    """Oracle: torch convolution of the undivided image (bf16-rounded operands, fp32 accumulation),
    cut back to this rank's tile."""
    from dist_utils import merge, split

    xg = merge(x_local.float(), cuts)
    w = layer.weight.detach().to(torch.bfloat16).float()
    b = None if layer.bias is None else layer.bias.detach().float()
    y = torch.nn.functional.conv2d(xg.to(torch.bfloat16).float(), w, b, padding=1)
    return split(y, cuts)


def _worker_recycled_halo_buffers(rank, world, mesh_shape):
    """Recycled padded buffers must not be overwritten by a neighbour that runs ahead.  Rank 1's
    convolution kernels start late; rank 0 runs two unchained layers in a forward-only loop, so its
    next halo push targets the buffer that rank 1 has not read yet.  Every iteration (different
    inputs) must match torch on the gathered image."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"sh": mesh_shape[0], "sw": mesh_shape[1], "col": 1})
    cuts = {2: mesh["sh"], 3: mesh["sw"]}
    torch.manual_seed(0)
    l1 = jb.modules.DistributedConv2d(64, 64, 3, dev, (mesh["sh"], mesh["sw"]), mesh["col"], padding=1)
    l2 = jb.modules.DistributedConv2d(64, 64, 3, dev, (mesh["sh"], mesh["sw"]), mesh["col"], padding=1)
    g = torch.Generator().manual_seed(7 + rank)
    xs = [torch.randn(1, 64, 40, 136, generator=g).to(dev) for _ in range(6)]
    if rank == 1:
        _delay_kernel("jb_conv3x3_c64", 30_000_000)          # about 15 ms per launch
    outs = []
    before = _lib.LAUNCHES
    from jigsaw_b200.ops.lazy_chain import materialize

    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for x in xs:
            y1 = materialize(l1(x))          # computed at once: two separate one-layer calls, not one chain
            outs.append((y1, materialize(l2(y1))))
    assert _lib.LAUNCHES > before, "the fused convolution did not run"
    torch.cuda.synchronize()
    symm.arena(dev).check_status(collective=True)
    for i, (x, (y1, y2)) in enumerate(zip(xs, outs)):
        r1 = _gathered_conv(x, l1, cuts, dev)
        assert_close(y1.float(), r1, f"iteration {i}: first layer", 0.0, 1e-2 * float(r1.abs().max()))
        r2 = _gathered_conv(y1.float(), l2, cuts, dev)
        assert_close(y2.float(), r2, f"iteration {i}: second layer", 0.0, 1e-2 * float(r2.abs().max()))


@pytest.mark.multigpu(2)
def test_recycled_halo_buffers_with_a_lagging_rank():
    run_distributed(_worker_recycled_halo_buffers, 2, (2, 1), backend="nccl", timeout=300)


def _worker_accumulation_with_a_lagging_rank(rank, world, mesh_shape):
    """Gradient accumulation under ``no_grad_sync`` has no collective between micro-batches that would
    keep the ranks in step: with rank 1's weight-gradient kernels delayed, the gradients accumulated by the
    fused chain over several micro-batches (summed over the ranks at the end) must equal those of the unfused
    torch + NCCL path."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.models import DomainCNN
    from jigsaw_b200.ops import symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"sh": mesh_shape[0], "sw": mesh_shape[1], "col": 1})
    torch.manual_seed(0)
    fused = DomainCNN(mesh, dev, depth=3)
    plain = DomainCNN(mesh, dev, depth=3, fuse=False)
    plain.load_state_dict(fused.state_dict())
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    g = torch.Generator().manual_seed(11 + rank)
    batches = [(torch.randn(1, 3, 40, 136, generator=g).to(dev), torch.randn(1, 3, 40, 136, generator=g).to(dev))
               for _ in range(4)]
    if rank == 1:
        _delay_kernel("jb_conv3x3_c64_wgrad", 30_000_000)
        _delay_kernel("jb_conv3x3_wgrad_thin", 30_000_000)
    fused.zero_grad()
    with jb.parallel.no_grad_sync():
        for x, y in batches:                       # no collective between the micro-batches
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = fused(x)
            loss_fn(out.float(), y).backward()
    jb.parallel.reduce_replica_grads(fused)        # one sum at the end, as a training loop does
    torch.cuda.synchronize()
    symm.arena(dev).check_status(collective=True)
    plain.zero_grad()
    with jb.parallel.no_grad_sync():
        for x, y in batches:
            loss_fn(plain(x), y).backward()
    jb.parallel.reduce_replica_grads(plain)
    # (the per-rank partial sums may differ between the two paths: the thin-channel weight gradient pairs
    # this rank's INPUT pixels with output-gradient pixels of its neighbours; the sums over the ranks agree)
    for (n, q), p in zip(plain.named_parameters(), fused.parameters()):
        assert_close(p.grad, q.grad, f"accumulated grad {n}", 0.0, 4e-2 * float(q.grad.abs().max()) + 1e-7)


@pytest.mark.multigpu(2)
def test_accumulation_with_a_lagging_rank():
    run_distributed(_worker_accumulation_with_a_lagging_rank, 2, (2, 1), backend="nccl", timeout=300)


def _worker_exact_halo(rank, world, mesh_shape):
    """Integer-valued inputs and weights: every product and sum is exact in fp32 and the bf16 rounding
    of the result is deterministic, so the fused layer must equal torch on the gathered image bit for
    bit; a wrong, stale or missing halo pixel cannot hide inside a tolerance."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from dist_utils import merge, split
    from jigsaw_b200.ops import symm

    torch.backends.cudnn.allow_tf32 = False
    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"sh": mesh_shape[0], "sw": mesh_shape[1], "col": 1})
    cuts = {2: mesh["sh"], 3: mesh["sw"]}
    layer = jb.modules.DistributedConv2d(64, 64, 3, dev, (mesh["sh"], mesh["sw"]), mesh["col"], padding=1)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        layer.weight.copy_(torch.randint(-1, 2, layer.weight.shape, generator=g).float())
        layer.bias.copy_(torch.randint(-3, 4, layer.bias.shape, generator=g).float())
    for it in range(3):
        xg = torch.randint(-2, 3, (2, 64, 40 * mesh_shape[0], 136 * mesh_shape[1]), generator=g).float().to(dev)
        x = split(xg, cuts)
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            y = layer(x)
        ref = torch.nn.functional.conv2d(xg, layer.weight.detach(), layer.bias.detach(), padding=1).to(torch.bfloat16)
        symm.arena(dev).check_status()
        ok = torch.equal(y, split(ref, cuts))
        from dist_utils import all_ok

        if not all_ok(ok):
            bad = (y.float() - split(ref, cuts).float()).abs()
            raise AssertionError(f"iteration {it}: rank {rank} differs at {int((bad > 0).sum())} elements, max {float(bad.max())}")


@pytest.mark.multigpu(2)
def test_exact_halo_two_gpus():
    run_distributed(_worker_exact_halo, 2, (2, 1), backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_exact_halo_four_gpus_with_corners():
    run_distributed(_worker_exact_halo, 4, (2, 2), backend="nccl", timeout=300)


def _worker_graphed_step(rank, world, mesh_shape):
    """A whole training step replayed as a CUDA graph must follow the eager run bit for bit
    (same kernels, same order), halo epochs included, and eager steps may follow replays."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.models import DomainCNN
    from jigsaw_b200.ops import symm
    from jigsaw_b200.utils import GraphedStep

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"sh": mesh_shape[0], "sw": mesh_shape[1], "col": 1})
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    g = torch.Generator().manual_seed(5 + rank)
    xs = [torch.randn(1, 3, 64, 136, generator=g).to(dev) for _ in range(4)]
    ys = [torch.randn(1, 3, 64, 136, generator=g).to(dev) for _ in range(4)]

    def make():
        torch.manual_seed(0)
        m = DomainCNN(mesh, dev, depth=4)
        o = torch.optim.Adam(m.parameters(), lr=1e-3, fused=True, capturable=True)

        def step(x, y):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = m(x)
            loss = loss_fn(out.float(), y)
            o.zero_grad(set_to_none=True)
            loss.backward()
            o.step()
            return loss

        return m, step

    side = torch.cuda.Stream(dev)
    order = [0, 0, 0, 0, 1, 2, 3]            # GraphedStep: 3 warm-up steps and one counting step on batch 0
    m1, eager = make()
    with torch.cuda.stream(side):
        ref = [float(eager(xs[i], ys[i])) for i in order]
    m2, step2 = make()
    xi, yi = xs[0].clone(), ys[0].clone()
    graphed = GraphedStep(step2, (xi, yi), warmup=3)
    assert graphed.launches_per_step > 0
    got = []
    for i in order[4:]:
        xi.copy_(xs[i])
        yi.copy_(ys[i])
        got.append(float(graphed.replay()))
    with torch.cuda.stream(side):
        after_ref, after_got = float(eager(xs[0], ys[0])), float(step2(xs[0], ys[0]))
    symm.arena(dev).check_status()
    assert got == ref[4:], (got, ref[4:])
    assert after_got == after_ref
    for p, q in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(p, q)
    graphed.close()


def test_graphed_step_one_gpu():
    run_distributed(_worker_graphed_step, 1, (1, 1), backend="nccl", timeout=300)


@pytest.mark.multigpu(2)
def test_graphed_step_two_gpus():
    run_distributed(_worker_graphed_step, 2, (2, 1), backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_graphed_step_four_gpus():
    run_distributed(_worker_graphed_step, 4, (2, 2), backend="nccl", timeout=300)


def _worker_graphed_vit(rank, world, mesh_shape, depth):
    """A transformer step (patch embedding, LayerNorm, gathered linear layers, ring attention, cross-entropy
    over sharded classes, replica gradient sums, fused Adam) replayed as a CUDA graph follows the eager run:
    the copy-engine pushes, their flags and every in-kernel exchange take their epochs from the replay counter."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.models import ViT, ViTConfig
    from jigsaw_b200.ops import _lib, symm
    from jigsaw_b200.optim import FusedAdam
    from jigsaw_b200.utils import GraphedStep

    dev = torch.device("cuda", rank)
    R, C = mesh_shape
    mesh = jb.make_process_mesh({"row": R, "col": C})
    row, col = mesh["row"], mesh["col"]
    # 128 tokens per row rank, one 64-wide head per column rank; 10 classes per column rank keep the tiny
    # classification head (8 rows) on the torch path
    cfg = ViTConfig(image_size=(64, 256), in_channels=4, patch=8, dim=128, heads=2, depth=depth, num_classes=20)
    loss_fn = jb.modules.DistributedCrossEntropyLoss(col, (row,))
    g = torch.Generator().manual_seed(11)
    xs, ys = [], []
    for _ in range(4):
        x = torch.randn(8, 4, 64, 256, generator=g)
        x = x[:, col.rank() * 4 // C:(col.rank() + 1) * 4 // C, :, row.rank() * 256 // R:(row.rank() + 1) * 256 // R]
        xs.append(x.contiguous().to(dev))
        ys.append(torch.randint(0, 20, (8,), generator=g).to(dev))

    def make():
        torch.manual_seed(3 + mesh["model"].rank())
        m = ViT(mesh, dev, cfg)
        o = FusedAdam(m.parameters(), lr=1e-3)

        def step(x, y):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = m(x)
            loss = loss_fn(out.float(), y)
            o.zero_grad(set_to_none=True)
            loss.backward()
            o.step()
            return loss

        return m, step

    side = torch.cuda.Stream(dev)
    order = [0, 0, 0, 0, 1, 2, 3, 1]
    m1, eager = make()
    with torch.cuda.stream(side):
        ref = [float(eager(xs[i], ys[i])) for i in order]
    m2, step2 = make()
    xi, yi = xs[0].clone(), ys[0].clone()
    before = _lib.dispatch_counts()
    graphed = GraphedStep(step2, (xi, yi), warmup=3)
    counts = _lib.dispatch_counts()
    for name in (("ring_attention",) if R > 1 else ()) + (("gather_linear",) if C > 1 else ()) + ("layer_norm",):
        assert counts.get(name, {}).get("fused", 0) > before.get(name, {}).get("fused", 0), (name, counts)
    got = []
    for i in order[4:]:
        xi.copy_(xs[i])
        yi.copy_(ys[i])
        got.append(float(graphed.replay()))
    torch.cuda.synchronize()
    symm.arena(dev).check_status()
    for a, b in zip(got, ref[4:]):
        assert abs(a - b) <= 2e-3 * abs(b), (got, ref[4:])
    for (n, p), q in zip(m1.named_parameters(), m2.parameters()):
        assert_close(q, p, f"graphed ViT: {n}", 2e-2, 2e-2)
    graphed.close()


@pytest.mark.multigpu(2)
def test_graphed_vit_step_ring_two_gpus():
    run_distributed(_worker_graphed_vit, 2, (2, 1), 2, backend="nccl", timeout=300)


@pytest.mark.multigpu(2)
def test_graphed_vit_step_gathered_linear_two_gpus():
    # depth 1 uses the staging ring of the gathered layers an odd number of times per step: the capture
    # then ends with the fence that separates consecutive replays
    run_distributed(_worker_graphed_vit, 2, (1, 2), 1, backend="nccl", timeout=300)


def _worker_layer_norm(rank, world):
    """LayerNorm over a feature dimension cut over two GPUs: the fused kernels (statistics
    exchanged through peer memory) against the undivided torch op, twice in a row and in both
    directions (the inbox halves alternate from launch to launch)."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"row": 1, "col": world})
    col = mesh["col"]
    torch.manual_seed(0)
    n = 256
    full = torch.nn.LayerNorm(n, device=dev)
    with torch.no_grad():
        full.weight.uniform_(0.5, 1.5)
        full.bias.normal_()
    ln = jb.modules.DistributedLayerNorm.convert_to_jigsaw(full, mesh, dev)
    for it, rows in enumerate((777, 777, 64)):
        x = torch.randn(rows, n, device=dev) * 3 + 1
        g = torch.randn(rows, n, device=dev)
        xl = x[:, rank * n // world:(rank + 1) * n // world].contiguous().requires_grad_(True)
        before = _lib.LAUNCHES
        y = ln(xl)
        assert _lib.LAUNCHES == before + 1
        y.backward(g[:, rank * n // world:(rank + 1) * n // world].contiguous())
        symm.arena(dev).check_status()
        xr = x.clone().requires_grad_(True)
        full.zero_grad()
        yr = full(xr)
        yr.backward(g)
        sl = slice(rank * n // world, (rank + 1) * n // world)
        assert_close(y.detach(), yr.detach()[:, sl], f"call {it}: output", 1e-4, 1e-4)
        assert_close(xl.grad, xr.grad[:, sl], f"call {it}: input gradient", 1e-4, 1e-4)
        assert_close(ln.weight.grad, full.weight.grad[sl], f"call {it}: weight gradient", 1e-4, 1e-3)
        assert_close(ln.bias.grad, full.bias.grad[sl], f"call {it}: bias gradient", 1e-4, 1e-3)
        ln.zero_grad()


@pytest.mark.multigpu(2)
def test_fused_layer_norm_two_gpus():
    run_distributed(_worker_layer_norm, 2, backend="nccl", timeout=300)


def _worker_cross_entropy(rank, world):
    """Cross-entropy over classes cut over two GPUs (partials exchanged inside the kernel) against
    the undivided torch op, for a trailing class dimension and for per-pixel classes."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"row": 1, "col": world})
    col = mesh["col"]
    torch.manual_seed(0)
    for shape in ((16, 1000), (2, 20, 24, 40), (16, 1000)):
        C = shape[1]
        x = torch.randn(*shape, device=dev) * 3
        t = torch.randint(0, C, (shape[0], *shape[2:]), device=dev)
        t.view(-1)[::5] = -100
        sl = slice(rank * C // world, (rank + 1) * C // world)
        xl = x[:, sl].contiguous().requires_grad_(True)
        before = _lib.LAUNCHES
        loss = jb.modules.functional.distributed_cross_entropy(xl, t, channel_group=col)
        loss.backward()
        assert _lib.LAUNCHES == before + 2
        symm.arena(dev).check_status()
        xr = x.clone().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(xr, t)
        ref.backward()
        assert_close(loss.detach(), ref.detach(), f"{shape}: loss", 1e-5, 1e-6)
        assert_close(xl.grad, xr.grad[:, sl], f"{shape}: gradient", 1e-4, 1e-6)


@pytest.mark.multigpu(2)
def test_fused_cross_entropy_two_gpus():
    run_distributed(_worker_cross_entropy, 2, backend="nccl", timeout=300)


def _worker_gather_linear(rank, world, mesh_axes):
    """DistributedLinear under bf16 autocast: the all-gather of the activations is fused into the
    tcgen05 GEMM (TMA loads from the peers' memory); forward and all gradients against the
    undivided fp32 layer, several layers in a row (the staging blocks alternate)."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh(mesh_axes)
    row, col = mesh["row"], mesh["col"]
    torch.manual_seed(0)
    dims = [256, 512, 256, 256]
    full = torch.nn.Sequential(*[torch.nn.Linear(dims[i], dims[i + 1], device=dev) for i in range(3)])
    layers = torch.nn.Sequential(*[jb.modules.DistributedLinear.convert_to_jigsaw(lin, mesh, dev) for lin in full])
    cuts = {0: row, 1: col}
    from dist_utils import split

    for it in range(2):
        x = torch.randn(512, 256, device=dev)
        g = torch.randn(512, 256, device=dev)
        xl = split(x, cuts).requires_grad_(True)
        before = _lib.LAUNCHES
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = layers(xl)
        assert _lib.LAUNCHES - before == 6, "three gathered GEMMs (publish + GEMM each) expected"
        y.backward(split(g, cuts).to(y.dtype))
        symm.arena(dev).check_status()
        xr = x.clone().requires_grad_(True)
        full.zero_grad()
        yr = full(xr)
        yr.backward(g)
        scale = float(yr.abs().max())
        assert_close(y.float(), split(yr.detach(), cuts), f"step {it}: output", 0.0, 3e-2 * scale)
        assert_close(xl.grad, split(xr.grad, cuts), f"step {it}: input gradient", 0.0, 3e-2 * float(xr.grad.abs().max()))
        for i, (a, b) in enumerate(zip(layers, full)):
            wg = split(b.weight.grad, {0: row if a.row_split > 1 else None, 1: col})
            assert_close(a.weight.grad, wg, f"step {it}: weight gradient {i}", 0.0, 3e-2 * float(b.weight.grad.abs().max()))
            assert_close(a.bias.grad, split(b.bias.grad, {0: col}), f"step {it}: bias gradient {i}", 0.0,
                         3e-2 * float(b.bias.grad.abs().max()))
        layers.zero_grad()


@pytest.mark.multigpu(2)
def test_gather_linear_two_gpus():
    run_distributed(_worker_gather_linear, 2, {"row": 1, "col": 2}, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_gather_linear_four_gpus():
    run_distributed(_worker_gather_linear, 4, {"row": 2, "col": 2}, backend="nccl", timeout=300)


def _worker_roll(rank, world, axes):
    """DistributedRoll on the fused kernel (elements stored straight into the neighbours' outputs)
    against torch.roll of the undivided tensor: several shifts (negative, larger than a tile),
    forward and backward, bf16 and fp32."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from dist_utils import merge, split
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh(axes)
    sh, sw = mesh["sh"], mesh["sw"]
    cuts = {1: sh, 2: sw}
    torch.manual_seed(0)
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(2, 16, 12, 8, device=dev).to(dtype)
        for shifts in ((3, -2), (-5, 4), (9, 0), (16, -7)):
            layer = jb.modules.DistributedRoll(shifts, (1, 2), (1, 2), (sh, sw), dev, dtype=dtype)
            xl = split(x, cuts).requires_grad_(True)
            before = _lib.LAUNCHES
            y = layer(xl)
            assert _lib.LAUNCHES == before + 1
            ref = torch.roll(x, shifts, (1, 2))
            assert torch.equal(y.detach(), split(ref, cuts)), (dtype, shifts)
            g = torch.randn_like(x)
            y.backward(split(g, cuts))
            assert torch.equal(xl.grad, split(torch.roll(g, tuple(-s for s in shifts), (1, 2)), cuts)), (dtype, shifts)
    symm.arena(dev).check_status()


@pytest.mark.multigpu(2)
def test_fused_roll_two_gpus():
    run_distributed(_worker_roll, 2, {"sh": 2, "sw": 1, "col": 1}, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_fused_roll_four_gpus():
    run_distributed(_worker_roll, 4, {"sh": 2, "sw": 2, "col": 1}, backend="nccl", timeout=300)


def _worker_group_norm(rank, world, axes):
    """GroupNorm of a volume tiled over GPUs on the fused kernels (grid barrier + in-kernel exchange
    between the tile ranks) against the undivided torch op."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from dist_utils import split
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh(axes)
    sh, sw = mesh["sh"], mesh["sw"]
    torch.manual_seed(0)
    full = torch.nn.GroupNorm(4, 16, device=dev)
    with torch.no_grad():
        full.weight.uniform_(0.5, 1.5)
        full.bias.normal_()
    gn = jb.modules.DistributedGroupNorm.convert_to_jigsaw(full, mesh, dev, row_kw="sh", spatial_group=(None, sh, sw))
    cuts = {3: sh, 4: sw}
    for it in range(3):
        x = torch.randn(2, 16, 6, 16, 8, device=dev) * 2 + it
        g = torch.randn(2, 16, 6, 16, 8, device=dev)
        xl = split(x, cuts).requires_grad_(True)
        before = _lib.LAUNCHES
        y = gn(xl)
        assert _lib.LAUNCHES == before + 1                 # one launch for the forward pass
        y.backward(split(g, cuts))
        # one for the backward pass, one for the sum of the weight / bias gradients over the tile ranks
        assert _lib.LAUNCHES == before + 3
        symm.arena(dev).check_status()
        xr = x.clone().requires_grad_(True)
        full.zero_grad()
        yr = full(xr)
        yr.backward(g)
        assert_close(y.detach(), split(yr.detach(), cuts), f"call {it}: output", 1e-4, 1e-4)
        assert_close(xl.grad, split(xr.grad, cuts), f"call {it}: input gradient", 1e-4, 1e-4)
        assert_close(gn.weight.grad, full.weight.grad, f"call {it}: weight gradient", 1e-4, 1e-3)
        assert_close(gn.bias.grad, full.bias.grad, f"call {it}: bias gradient", 1e-4, 1e-3)
        gn.zero_grad()


@pytest.mark.multigpu(2)
def test_fused_group_norm_two_gpus():
    run_distributed(_worker_group_norm, 2, {"sh": 2, "sw": 1, "col": 1}, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_fused_group_norm_four_gpus():
    run_distributed(_worker_group_norm, 4, {"sh": 2, "sw": 2, "col": 1}, backend="nccl", timeout=300)


def _worker_all_to_all(rank, world):
    """The re-sharding all-to-all on the peer-memory kernel (Ulysses' sequence <-> head exchange):
    against a reference assembled from an all-gather, its inverse, and through autograd."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist

    import jigsaw_b200 as jb
    from jigsaw_b200._core.collectives import all_to_all_dims
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"row": world, "col": 1})
    group = mesh["row"]
    torch.manual_seed(rank)
    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(3, 2, 6, 4 * world, 16, device=dev).to(dtype)            # (3, b, s/P, h, d)
        everyone = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(everyone, x, group=group)
        h = x.shape[-2] // world
        expect = torch.cat([e[..., rank * h:(rank + 1) * h, :] for e in everyone], dim=-3)   # (3, b, s, h/P, d)
        before = _lib.LAUNCHES
        xg = x.clone().requires_grad_(True)
        y = all_to_all_dims(xg, group, split_dim=-2, cat_dim=-3)
        assert _lib.LAUNCHES == before + 1
        assert torch.equal(y.detach(), expect)
        back = all_to_all_dims(y, group, split_dim=-3, cat_dim=-2)
        assert torch.equal(back.detach(), x)
        back.backward(torch.ones_like(back))
        assert torch.equal(xg.grad, torch.ones_like(x))
    symm.arena(dev).check_status()


@pytest.mark.multigpu(2)
def test_fused_all_to_all_two_gpus():
    run_distributed(_worker_all_to_all, 2, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_fused_all_to_all_four_gpus():
    run_distributed(_worker_all_to_all, 4, backend="nccl", timeout=300)


def _worker_ring_attention(rank, world):
    """Ring attention whose key / value chunks are pulled from their owners' memory by the peer-fetch
    kernel (side stream, next chunk in flight while the current one is attended to) against the
    undivided attention layer: output and every gradient."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from dist_utils import split
    from jigsaw_b200.modules.attention import Attention
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"row": world, "col": 1})
    torch.manual_seed(0)
    serial = Attention(64, 64, 64, 4, dev, attn_backend="math")
    ring = Attention.convert_to_jigsaw(serial, mesh, dev, ring=True, attn_backend="math")
    for it in range(2):
        x = torch.randn(2, 32 * world, 64, device=dev)
        g = torch.randn(2, 32 * world, 64, device=dev)
        xl = split(x, {1: mesh["row"]}).requires_grad_(True)
        before = _lib.LAUNCHES
        y = ring(xl)
        assert _lib.LAUNCHES > before, "the peer-fetch kernels did not run"
        y.backward(split(g, {1: mesh["row"]}))
        symm.arena(dev).check_status()
        xr = x.clone().requires_grad_(True)
        serial.zero_grad()
        yr = serial(xr)
        yr.backward(g)
        # on CUDA the attention core computes in half precision even for fp32 inputs: compare at that level
        tol = 2e-2
        assert_close(y.detach(), split(yr.detach(), {1: mesh["row"]}), f"call {it}: output", 0.0, tol * float(yr.detach().abs().max()))
        assert_close(xl.grad, split(xr.grad, {1: mesh["row"]}), f"call {it}: input gradient", 0.0, tol * float(xr.grad.abs().max()))
        for (n, p), q in zip(ring.named_parameters(), serial.parameters()):
            assert_close(p.grad, q.grad, f"call {it}: gradient of {n}", 0.0, tol * float(q.grad.abs().max()))
        ring.zero_grad()


@pytest.mark.multigpu(2)
def test_ring_attention_peer_fetch_two_gpus():
    run_distributed(_worker_ring_attention, 2, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_ring_attention_peer_fetch_four_gpus():
    run_distributed(_worker_ring_attention, 4, backend="nccl", timeout=300)


def _worker_ulysses_qkv(rank, world):
    """Ulysses attention under bf16 autocast: the sequence -> head exchange rides in the epilogue of the
    QKV projection GEMM (tiles stored into the destination ranks' inboxes), against the undivided
    attention layer: output and every gradient."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from dist_utils import split
    from jigsaw_b200.modules.attention import Attention
    from jigsaw_b200.ops import _lib, symm, ulysses_fused

    ulysses_fused.FUSE_QKV_PROJECTION = ulysses_fused.FUSE_OUTPUT_PROJECTION = True
    dev = torch.device("cuda", rank) if torch.cuda.is_available() else torch.device("cpu")
    mesh = jb.make_process_mesh({"row": world, "col": 1})
    torch.manual_seed(0)
    serial = Attention(128, 256, 128, 4, dev, attn_backend="math")
    uly = Attention.convert_to_jigsaw(serial, mesh, dev, ring=False, ulysses=True, attn_backend="math")
    for it in range(3):
        x = torch.randn(2, 96 * world, 128, device=dev)
        g = torch.randn(2, 96 * world, 128, device=dev)
        xl = split(x, {1: mesh["row"]}).requires_grad_(True)
        before = _lib.LAUNCHES
        with torch.autocast(dev.type, dtype=torch.bfloat16):
            y = uly(xl)
        if dev.type == "cuda":
            assert _lib.LAUNCHES >= before + 5, "the fused projections did not run"
        y.float().backward(split(g, {1: mesh["row"]}))
        if dev.type == "cuda":
            symm.arena(dev).check_status()
        xr = x.clone().requires_grad_(True)
        serial.zero_grad()
        yr = serial(xr)
        yr.backward(g)
        tol = 3e-2
        assert_close(y.detach().float(), split(yr.detach(), {1: mesh["row"]}), f"call {it}: output", 0.0, tol * float(yr.detach().abs().max()))
        assert_close(xl.grad, split(xr.grad, {1: mesh["row"]}), f"call {it}: input gradient", 0.0, tol * float(xr.grad.abs().max()))
        for (n, p), q in zip(uly.named_parameters(), serial.parameters()):
            assert_close(p.grad, q.grad, f"call {it}: gradient of {n}", 0.0, tol * float(q.grad.abs().max()))
        uly.zero_grad()


@pytest.mark.multigpu(2)
def test_ulysses_fused_projection_two_gpus():
    run_distributed(_worker_ulysses_qkv, 2, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_ulysses_fused_projection_four_gpus():
    run_distributed(_worker_ulysses_qkv, 4, backend="nccl", timeout=300)


def _worker_ring_flash_attention(rank, world):
    """Ring attention as one fused launch: keys / values (backward: queries, output gradients, log-sum-exp,
    D) are pulled by TMA from the owners' memory.  Output and the three gradients of the local sequence
    part against fp32 attention over the gathered sequence; several calls in a row (the staging blocks
    alternate) with different data."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from dist_utils import merge
    from jigsaw_b200.ops import _lib, attention_fused, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"row": world, "col": 1})
    group = mesh["row"]
    b, h, s = 2, 3, 384
    gen = torch.Generator().manual_seed(50 + rank)
    for it in range(3):
        q, k, v, g = (torch.randn(b, h, s, 64, generator=gen).to(dev).bfloat16() for _ in range(4))
        ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
        before = _lib.LAUNCHES
        with _lib.strict_fused():
            out = attention_fused.maybe_fused_ring_attention(ql, kl, vl, 0.125, group)
        assert _lib.LAUNCHES - before == 2, "one publish and ONE attention launch for the whole ring"
        out.backward(g)
        symm.arena(dev).check_status(collective=True)
        cuts = {2: group}
        qa, ka, va, ga = (merge(t.float(), cuts).requires_grad_(True) for t in (q, k, v, g))
        ref = torch.softmax(0.125 * (qa @ ka.transpose(-1, -2)), dim=-1) @ va
        ref.backward(ga.detach())
        sl = slice(rank * s, (rank + 1) * s)
        assert_close(out.float(), ref.detach()[:, :, sl], f"call {it}: output", 0.0, 2e-2 * float(ref.abs().max()))
        for name, mine, full in (("dq", ql.grad, qa.grad), ("dk", kl.grad, ka.grad), ("dv", vl.grad, va.grad)):
            assert_close(mine.float(), full[:, :, sl], f"call {it}: {name}", 0.0, 2e-2 * float(full.abs().max()))


@pytest.mark.multigpu(2)
def test_ring_flash_attention_two_gpus():
    run_distributed(_worker_ring_flash_attention, 2, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_ring_flash_attention_four_gpus():
    run_distributed(_worker_ring_flash_attention, 4, backend="nccl", timeout=300)


def _worker_all_reduce_kernel(rank, world):
    """The peer-memory all-reduce kernel against NCCL on integer-valued data (every partial sum is exact, so
    the results must agree bit for bit): whole world and sub-groups, several sizes, twice in a row, and
    through the overlapped reducer on its side stream."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist

    from jigsaw_b200.ops import _lib, reduce_fused, symm

    dev = torch.device("cuda", rank)
    groups = [(list(range(world)), dist.group.WORLD)]
    if world == 4:
        for members in ([0, 1], [2, 3], [0, 2], [1, 3]):
            g = dist.new_group(members)
            if rank in members:
                groups.append((members, g))
    gen = torch.Generator().manual_seed(rank)
    for ranks, pg in groups:
        for it, sizes in enumerate(((36928,), (5, 1733, 64), (1 << 20, 3), (36928,))):
            ts = [torch.randint(-50, 50, (n,), generator=gen).float().to(dev) for n in sizes]
            ref = [t.clone() for t in ts]
            for r in ref:
                dist.all_reduce(r, group=pg)
            before = _lib.LAUNCHES
            with _lib.strict_fused():
                assert reduce_fused.maybe_fused_all_reduce(ts, ranks)
            assert _lib.LAUNCHES == before + 1
            for t, r in zip(ts, ref):
                assert torch.equal(t, r), (ranks, it)
    # side stream: reductions of several buckets in flight while the main stream keeps working
    red = reduce_fused.OverlappedReducer(dev, list(range(world)), scale=0.5)
    buckets = [[torch.randint(-9, 9, (4000 + 100 * i,), generator=gen).float().to(dev), torch.randint(-9, 9, (64,), generator=gen).float().to(dev)]
               for i in range(5)]
    refs = [[t.clone() for t in b] for b in buckets]
    busy = torch.randn(2048, 2048, device=dev)
    for b in buckets:
        red.add(b)
        busy = busy @ busy * 1e-3
    red.finish()
    for b, rb in zip(buckets, refs):
        for t, r in zip(b, rb):
            dist.all_reduce(r)
            assert torch.equal(t, r * 0.5)
    symm.arena(dev).check_status(collective=True)


@pytest.mark.multigpu(2)
def test_all_reduce_kernel_two_gpus():
    run_distributed(_worker_all_reduce_kernel, 2, backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_all_reduce_kernel_four_gpus():
    run_distributed(_worker_all_reduce_kernel, 4, backend="nccl", timeout=300)


def _worker_fused_softmax(rank, world):
    """Softmax and log-softmax over a class dimension cut over the GPUs (row statistics exchanged inside the
    kernel, gradient row sums through the peer-memory all-reduce) against the undivided torch ops: trailing
    and inner class dimensions, fp32 and bf16, forward and backward; and the single-GPU form of the same kernels."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib, softmax_fused, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"row": 1, "col": world})
    col = mesh["col"]
    torch.manual_seed(0)
    for shape, dim in (((16, 1000), 1), ((2, 20, 24, 40), 1), ((3, 5, 128), -1)):
        for dtype in (torch.float32, torch.bfloat16):
            for log in (False, True):
                x = (torch.randn(*shape, device=dev) * 3).to(dtype)
                g = torch.randn(*shape, device=dev)
                C = shape[dim]
                sl = [slice(None)] * len(shape)
                sl[dim] = slice(rank * C // world, (rank + 1) * C // world)
                xl = x[tuple(sl)].contiguous().requires_grad_(True)
                fn = jb.modules.functional.distributed_log_softmax if log else jb.modules.activation.distributed_softmax
                before = _lib.LAUNCHES
                with _lib.strict_fused():
                    y = fn(xl, dim, col)
                assert _lib.LAUNCHES == before + 2
                y.backward(g[tuple(sl)].to(y.dtype))
                symm.arena(dev).check_status()
                xr = x.float().requires_grad_(True)
                ref = torch.log_softmax(xr, dim) if log else torch.softmax(xr, dim)
                ref.backward(g)
                tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
                assert_close(y.float(), ref.detach()[tuple(sl)], f"{shape} {dtype} log={log}: output", tol, tol)
                assert_close(xl.grad.float(), xr.grad[tuple(sl)], f"{shape} {dtype} log={log}: gradient", tol, tol * max(float(xr.grad.abs().max()), 1e-3))
    # one GPU, no group: the same kernels without an exchange
    x = torch.randn(7, 300, device=dev, requires_grad=True)
    y = softmax_fused.maybe_fused_softmax(x, -1, None, log=False)
    y.backward(torch.ones_like(y) * torch.arange(300, device=dev))
    xr = x.detach().clone().requires_grad_(True)
    torch.softmax(xr, -1).backward(torch.ones_like(y) * torch.arange(300, device=dev))
    assert_close(y, torch.softmax(xr, -1).detach(), "local softmax", 1e-5, 1e-6)
    assert_close(x.grad, xr.grad, "local softmax gradient", 1e-4, 1e-5)


@pytest.mark.multigpu(2)
def test_fused_softmax_two_gpus():
    run_distributed(_worker_fused_softmax, 2, backend="nccl", timeout=300)


def _worker_overlapped_grad_sync(rank, world):
    """``OverlappedGradSync`` on GPUs: buckets reduced by the peer-memory all-reduce on a side stream give the
    gradients of the in-graph mode bit for bit (integer-valued data: every sum is exact)."""
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"sh": world, "sw": 1, "col": 1})
    M = jb.modules

    def build():
        torch.manual_seed(0)
        model = torch.nn.Sequential(M.DistributedConv2d(2, 4, 3, dev, (mesh["sh"], mesh["sw"]), mesh["col"], padding=1),
                                    M.DistributedConv2d(4, 2, 3, dev, (mesh["sh"], mesh["sw"]), mesh["col"], padding=1))
        with torch.no_grad():
            for i, p in enumerate(model.parameters()):
                p.copy_(torch.randint(-2, 3, p.shape, generator=torch.Generator().manual_seed(100 + i)).float())
        return model

    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randint(-2, 3, (1, 2, 8, 8), generator=g).float().to(dev)
    gy = torch.randint(-2, 3, (1, 2, 8, 8), generator=g).float().to(dev)
    ref = build()
    ref(x).backward(gy)
    for bucket_bytes in (1, 1 << 20):
        model = build()
        before = _lib.dispatch_counts().get("all_reduce", {}).get("fused", 0)
        launches = _lib.LAUNCHES
        with jb.parallel.OverlappedGradSync(model, bucket_bytes=bucket_bytes) as sync:
            model(x).backward(gy)
        torch.cuda.synchronize()
        symm.arena(dev).check_status(collective=True)
        assert sync.launched >= 1 and _lib.LAUNCHES - launches >= sync.launched, "the buckets must go through the own all-reduce kernel"
        assert _lib.dispatch_counts().get("all_reduce", {}).get("fused", 0) == before, "no blocking in-graph reduction inside the context"
        for (n, p), q in zip(model.named_parameters(), ref.parameters()):
            assert all_ok(torch.equal(p.grad, q.grad)), f"bucket {bucket_bytes}: {n}"


@pytest.mark.multigpu(2)
def test_overlapped_grad_sync_two_gpus():
    run_distributed(_worker_overlapped_grad_sync, 2, backend="nccl", timeout=300)
