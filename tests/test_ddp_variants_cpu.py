"""Library layers under ``DistributedDataParallel`` over the ``dp`` axis, every way of wrapping.

For each layer kind and each DDP variant the gradient of a replicated parameter must be
``AVG_dp(SUM_replicas(local))`` and that of a sharded parameter ``AVG_dp(local)``, where ``local`` is
what the same rank computes with the in-graph reduction switched off; the expectation is assembled
from those per-rank quantities with explicit collectives, independently of the code under test.
Linear and convolution cells run on small integers, so every sum is exact and the comparison is
bitwise; attention and layer norm are compared to a tight tolerance.  Replicas must hold identical
bits in every case.

Reference behaviours covered: tests/test_ddp.py:32-49 (the variant list), :215-258 (the composition
check), :261-272 (mutation: the matrix notices a missing reduction), :275-295 (joint groups).
"""

import contextlib

import pytest
import torch

from dist_utils import all_ok, run_distributed

KINDS = ("linear", "conv_halo", "conv_patchify", "attention", "layer_norm")
EXACT = {"linear", "conv_halo", "conv_patchify"}
VARIANTS = ("no_ddp", "ddp", "bucket_view", "find_unused", "static_graph", "fp16_hook", "no_sync",
            "joint", "joint_bucket_view", "joint_static_graph", "joint_fp16", "joint_no_sync", "joint_accum")


def _ints(shape, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-2, 3, tuple(shape), generator=g).to(dtype)


def _build(kind, mesh):
    import jigsaw_b200 as jb
    import torch.distributed as dist

    M = jb.modules
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    R, C = row.size(), col.size()
    if kind == "linear":
        layer = M.DistributedLinear(8, 8, "cpu", model, row, col)
        shape = (2, 4 // R, 8 // C)
    elif kind == "conv_halo":
        layer = M.DistributedConv2d(4, 4, 3, "cpu", row, col, padding=1)
        shape = (2, 4 // C, 4, 8 // R)
    elif kind == "conv_patchify":
        layer = M.DistributedConv2d(4, 4, 2, "cpu", row, col, stride=2)
        shape = (2, 4 // C, 4, 8 // R)
    elif kind == "attention":
        layer = M.DistributedAttention(8, 8, 8, 2, col.rank(), "cpu", row, col, qk_norm=True, attn_backend="math")
        shape = (2, 8 // R, 8 // C)
    else:
        layer = M.DistributedLayerNorm(8, model.rank(), "cpu", row, col)
        shape = (2, 8 // R, 8 // C)
    with torch.no_grad():
        for i, p in enumerate(layer.parameters()):
            if kind in EXACT:
                p.copy_(_ints(p.shape, 1000 + i, p.dtype))          # the same small integers on every rank
    if kind not in EXACT:
        jb.parallel.broadcast_replicas(layer)
        for p in layer.parameters():                               # and the same over dp
            dist.broadcast(p.data, dist.get_process_group_ranks(mesh["dp"])[0], group=mesh["dp"])

    def make_input(step):
        seed = 10 * dist.get_rank() + step
        if kind in EXACT:
            return _ints(shape, seed)
        return torch.randn(shape, generator=torch.Generator().manual_seed(seed))

    return layer, make_input


def _wrap(layer, variant, mesh):
    import jigsaw_b200 as jb
    from torch.distributed.algorithms.ddp_comm_hooks import default_hooks
    from torch.nn.parallel import DistributedDataParallel as DDP

    if variant == "no_ddp":
        return layer
    joint = variant.startswith("joint")
    base = variant.removeprefix("joint_") if joint else variant
    kwargs = {"bucket_view": {"gradient_as_bucket_view": True}, "find_unused": {"find_unused_parameters": True},
              "static_graph": {"static_graph": True}}.get(base, {})
    ddp = DDP(layer, process_group=mesh["dp"], **kwargs)
    if variant == "fp16_hook":
        ddp.register_comm_hook(mesh["dp"], default_hooks.fp16_compress_hook)
    if joint:
        jb.parallel.register_joint_comm_hook(ddp, default_hooks.fp16_compress_wrapper if base == "fp16" else None)
    return ddp


def _step(model, make_input, n_micro, no_sync=False):
    import torch.distributed as dist

    for step in range(n_micro):
        ctx = model.no_sync() if no_sync and step < n_micro - 1 else contextlib.nullcontext()
        with ctx:
            y = model(make_input(step))
            y.backward(_ints(y.shape, 500 + 10 * dist.get_rank() + step))


@contextlib.contextmanager
def _sync_off():
    from jigsaw_b200.parallel import _sync

    old = _sync._SYNC_DISABLED
    _sync._SYNC_DISABLED = True
    try:
        yield
    finally:
        _sync._SYNC_DISABLED = old


def _expected(layer, make_input, n_micro, mesh, ddp):
    import jigsaw_b200 as jb
    import torch.distributed as dist

    with _sync_off():
        _step(layer, make_input, n_micro)
    local = [p.grad.clone() for p in layer.parameters()]
    layer.zero_grad(set_to_none=True)
    out = []
    for p, g in zip(layer.parameters(), local):
        for grp in jb.parallel.replica_groups(p):
            dist.all_reduce(g, group=grp)
        if ddp and mesh["dp"].size() > 1:
            g /= mesh["dp"].size()
            dist.all_reduce(g, group=mesh["dp"])
        out.append(g)
    return out


def _identical_over(t, group):
    import torch.distributed as dist

    parts = [torch.empty_like(t) for _ in range(group.size())]
    dist.all_gather(parts, t.contiguous(), group=group)
    return all(torch.equal(p, parts[0]) for p in parts)


def _worker_matrix(rank, world, axes, kinds, variants):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh(dict(axes), model_parallel_axes=("row", "col"))
    for kind in kinds:
        for variant in variants:
            layer, make_input = _build(kind, mesh)
            n_micro = 2 if variant in ("no_sync", "joint_no_sync", "joint_accum") else 1
            expected = _expected(layer, make_input, n_micro, mesh, ddp=variant != "no_ddp")
            wrapped = _wrap(layer, variant, mesh)
            _step(wrapped, make_input, n_micro, no_sync=variant in ("no_sync", "joint_no_sync"))
            tag = f"{dict(axes)} {kind} {variant}"
            for (name, p), e in zip(layer.named_parameters(), expected):
                assert p.grad is not None, f"{tag}: {name} has no gradient"
                if kind in EXACT:
                    ok = torch.equal(p.grad, e)
                else:
                    loose = variant in ("fp16_hook", "joint_fp16")
                    scale = float(e.abs().max())
                    ok = torch.allclose(p.grad, e, rtol=1e-2 if loose else 1e-5, atol=max((2e-3 if loose else 1e-4) * scale, 1e-6))
                assert all_ok(ok), f"{tag}: gradient of {name} is not AVG_dp(SUM_replicas(local))"
                for grp in jb.parallel.replica_groups(p):
                    assert all_ok(_identical_over(p.grad, grp)), f"{tag}: {name}.grad differs between replicas"
                if variant != "no_ddp":
                    assert all_ok(_identical_over(p.grad, mesh["dp"])), f"{tag}: {name}.grad differs over dp"


@pytest.mark.parametrize("axes", [(("dp", 2), ("row", 2), ("col", 2)), (("dp", 2), ("row", 2), ("col", 1)),
                                  (("dp", 4), ("row", 1), ("col", 1)), (("dp", 1), ("row", 2), ("col", 2))],
                         ids=["2x2x2", "2x2x1", "4x1x1", "1x2x2"])
def test_ddp_composition_matrix(axes):
    world = 1
    for _, n in axes:
        world *= n
    run_distributed(_worker_matrix, world, axes, KINDS, VARIANTS, timeout=900)


def _worker_mutation(rank, world):
    """With the in-graph reduction off under plain DDP the matrix's comparison must fail."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"dp": 2, "row": 2, "col": 1}, model_parallel_axes=("row", "col"))
    layer, make_input = _build("conv_halo", mesh)
    expected = _expected(layer, make_input, 1, mesh, ddp=True)
    wrapped = _wrap(layer, "ddp", mesh)
    with _sync_off():
        _step(wrapped, make_input, 1)
    same = all(torch.equal(p.grad, e) for p, e in zip(layer.parameters(), expected))
    assert all_ok(not same), "the gradients matched although the reduction over the tile ranks was off"


def test_missing_reduction_is_noticed():
    run_distributed(_worker_mutation, 4, timeout=300)


def _worker_joint_groups(rank, world):
    """Under the joint hook every parameter is averaged over exactly the ranks that hold a copy of it."""
    import jigsaw_b200 as jb
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    mesh = jb.make_process_mesh({"dp": 2, "row": 2, "col": 2}, model_parallel_axes=("row", "col"))
    layer, make_input = _build("linear", mesh)           # weight sharded, bias replicated over the row ranks
    ddp = DDP(layer, process_group=mesh["dp"])
    state = jb.parallel.register_joint_comm_hook(ddp)
    dp_ranks = set(dist.get_process_group_ranks(mesh["dp"]))
    assert any(jb.parallel.replica_groups(p) for p in layer.parameters())
    for name, p in layer.named_parameters():
        got = set(dist.get_process_group_ranks(state.group_of(p)))
        assert dist.get_rank() in got, name
        if jb.parallel.replica_groups(p):
            row = set(dist.get_process_group_ranks(mesh["row"]))
            assert len(got) == mesh["dp"].size() * mesh["row"].size() and dp_ranks <= got and row <= got, (name, got)
        else:
            assert got == dp_ranks, (name, got)
    # a state whose hook was never registered would scale without summing: refused in the first forward
    other, _ = _build("conv_halo", mesh)
    bare = DDP(other, process_group=mesh["dp"])
    jb.parallel.JointCommHookState(bare)
    with pytest.raises(RuntimeError, match="not registered"):
        bare(make_input(0).new_zeros(2, 2, 4, 4))


def test_joint_hook_groups_and_unregistered_state():
    run_distributed(_worker_joint_groups, 8, timeout=300)
