"""Guards around data parallelism: DDP over a group that spans model-parallel ranks is refused, library modules
start with identical replicas whatever the seeds, diverged replicas are caught (by DDP's first forward and by
``assert_replica_consistency`` on every rank), ``wrap_ddp`` repairs them first, re-sharding moves the replica marks
onto the new groups, and plain layers without a mark are reported.

Reference behaviours covered: tests/test_ddp_guards.py:35-63 (group checks), :64-80 (identical replicas at
construction), :81-108 (divergence before DDP, ``wrap_ddp``), :110-130 (consistency check on every rank), :131-160
(re-marking after a re-shard), :162-215 (unmarked plain layers), :216-234 (plain submodules of library modules).
"""

import pytest
import torch

from dist_utils import all_ok, run_distributed
from test_ddp_variants_cpu import KINDS, _build, _expected, _ints


def _mesh(dp, row, col):
    import jigsaw_b200 as jb

    return jb.make_process_mesh({"dp": dp, "row": row, "col": col}, model_parallel_axes=("row", "col"))


def _perturb(p):
    with torch.no_grad():
        p.add_(1.0)


def _worker_groups(rank, world):
    import jigsaw_b200 as jb
    from torch.nn.parallel import DistributedDataParallel as DDP

    mesh = _mesh(2, 2, 1)
    for kind in ("linear", "conv_halo", "attention"):
        layer, make_input = _build(kind, mesh)
        ddp = DDP(layer)                                        # the default group spans the row axis
        with pytest.raises(RuntimeError, match="spans model-parallel"):
            ddp(make_input(0))
        with pytest.raises(RuntimeError, match="spans model-parallel"):
            jb.parallel.check_ddp(ddp)
    layer, make_input = _build("conv_halo", mesh)
    ddp = DDP(layer, process_group=mesh["dp"])
    ddp(make_input(0)).sum().backward()
    # on a pure data-parallel mesh the default group IS the dp axis
    pure = _mesh(4, 1, 1)
    layer, make_input = _build("conv_halo", pure)
    DDP(layer)(make_input(0)).sum().backward()
    # DDP broadcasts over dp only: replicas that differ inside a model copy stay so, and the first forward says it
    layer, make_input = _build("conv_halo", mesh)
    if rank == 1:
        _perturb(layer.weight)
    ddp = DDP(layer, process_group=mesh["dp"])
    with pytest.raises(RuntimeError, match="differ across their replica groups"):
        ddp(make_input(0))
    # wrap_ddp broadcasts the replicas first
    layer, make_input = _build("conv_halo", mesh)
    if rank == 1:
        _perturb(layer.weight)
    ddp = jb.parallel.wrap_ddp(layer, mesh)
    jb.debug.assert_replica_consistency(layer, mesh)
    ddp(make_input(0)).sum().backward()
    with pytest.raises(TypeError):
        jb.parallel.wrap_ddp(layer, mesh, process_group=mesh["dp"])


def test_group_checks_and_diverged_replicas():
    run_distributed(_worker_groups, 4, timeout=300)


def _worker_replicas(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist
    from jigsaw_b200.parallel._replicas import replica_divergence
    from torch.nn.parallel import DistributedDataParallel as DDP

    mesh = _mesh(2, 2, 2)
    every = list({id(g): g for g in mesh.values()}.values())
    # 1. library modules broadcast their replicas when they are built: a different seed on every rank does not matter
    for kind in KINDS:
        torch.manual_seed(1234 + rank)
        M = jb.modules
        row, col, model = mesh["row"], mesh["col"], mesh["model"]
        layer = {"linear": lambda: M.DistributedLinear(8, 8, "cpu", model, row, col),
                 "conv_halo": lambda: M.DistributedConv2d(4, 4, 3, "cpu", row, col, padding=1),
                 "conv_patchify": lambda: M.DistributedConv2d(4, 4, 2, "cpu", row, col, stride=2),
                 "attention": lambda: M.DistributedAttention(8, 8, 8, 2, col.rank(), "cpu", row, col, qk_norm=True, attn_backend="math"),
                 "layer_norm": lambda: M.DistributedLayerNorm(8, model.rank(), "cpu", row, col)}[kind]()
        assert any(jb.parallel.replica_groups(p) for p in layer.parameters()), kind
        div = replica_divergence([(p, jb.parallel.replica_groups(p)) for p in layer.parameters()])
        for g in every:
            dist.all_reduce(div, op=dist.ReduceOp.MAX, group=g)
        assert not div.any(), (kind, [n for (n, _), d in zip(layer.named_parameters(), div.tolist()) if d > 0])
    # 2. the consistency check fails on EVERY rank, names the parameter, and honours atol
    for axis in ("replica", "dp"):
        layer, _ = _build("attention", mesh)
        jb.debug.assert_replica_consistency(layer, mesh)
        name, p = next((n, q) for n, q in layer.named_parameters() if jb.parallel.replica_groups(q))
        if (axis == "replica" and rank == 7) or (axis == "dp" and mesh["dp"].rank() == 1):
            _perturb(p)                                       # one rank of one copy / one whole copy, consistently
        with pytest.raises(AssertionError, match=name.replace(".", r"\.")):
            jb.debug.assert_replica_consistency(layer, mesh)
        with pytest.raises(AssertionError):
            jb.debug.assert_replica_consistency(layer, mesh, atol=0.5)
        jb.debug.assert_replica_consistency(layer, mesh, atol=1.001)    # the perturbation is 1 up to float32 rounding
    # 3. after re-sharding, the marks sit on the new groups and the gradient is summed over the new spatial group
    old, new = mesh, _mesh(2, 4, 1)
    conv = jb.modules.DistributedConv2d(4, 4, 3, "cpu", old["row"], old["col"], padding=1)
    with torch.no_grad():
        for i, p in enumerate(conv.parameters()):
            p.copy_(_ints(p.shape, 1000 + i))
    conv.reshard_parameters(old, new)
    for p in conv.parameters():
        assert jb.parallel.replica_groups(p) == (new["row"],)

    def make_input(step):
        return _ints((2, 4, 4, 2), 10 * rank + step)

    expected = _expected(conv, make_input, 1, new, ddp=True)
    ddp = jb.parallel.wrap_ddp(conv, new)
    y = ddp(make_input(0))
    y.backward(_ints(y.shape, 500 + 10 * rank))
    for (name, p), e in zip(conv.named_parameters(), expected):
        assert all_ok(torch.equal(p.grad, e)), f"after the re-shard: {name}"
    # 4. a plain layer behind a library layer, replicated over all model ranks: without a mark it drifts,
    #    and only unmarked=True sees that; the sharded conv weight is never reported
    for mark in (False, True):
        class Net(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.conv = jb.modules.DistributedConv2d(4, 4, 3, "cpu", mesh["row"], mesh["col"], padding=1)
                self.head = torch.nn.Linear(4, 4)
                with torch.no_grad():
                    for i, p in enumerate(self.parameters()):
                        p.copy_(_ints(p.shape, 1000 + i))
                if mark:
                    for p in self.head.parameters():
                        jb.parallel.mark_replicated(p, mesh["model"])

            def forward(self, x):
                return jb.parallel.synced_call(self.head, self.conv(x))

        net = Net()
        ddp = DDP(net, process_group=mesh["dp"])
        opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
        ddp(_ints((2, 2, 4, 4), 10 * rank)).pow(2).mean().backward()
        opt.step()
        jb.debug.assert_replica_consistency(net, mesh)         # blind to the missing mark
        if mark:
            jb.debug.assert_replica_consistency(net, mesh, unmarked=True)
        else:
            with pytest.raises(AssertionError, match="carry no replica mark") as err:
                jb.debug.assert_replica_consistency(net, mesh, unmarked=True)
            assert "head.weight" in str(err.value) and "conv.weight" not in str(err.value)
    # 5. a plain submodule INSIDE a library module is that module's to shard: never reported as unmarked
    norm = jb.modules.DistributedGroupNorm(4, 8, "cpu", channel_group=mesh["col"])
    norm.inner = torch.nn.Linear(2, 2)
    with torch.no_grad():
        norm.weight.fill_(1.0 + mesh["col"].rank())
        norm.inner.weight.fill_(1.0 + mesh["col"].rank())
        norm.inner.bias.zero_()
        norm.bias.zero_()
    jb.debug.assert_replica_consistency(norm, mesh, unmarked=True)


def test_replicas_consistency_remarking_and_unmarked_layers():
    run_distributed(_worker_replicas, 8, timeout=600)
