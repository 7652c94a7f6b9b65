"""``DistributedLinear`` beyond plain parity: summed losses (an expanded, stride-0 upstream gradient) on every
gradient path and transport, the column-only layout (``model_group == col_group``: weight replicated over the rows)
with its conversions, re-sharding between the two layouts and the replica marks that follow, bias initialisation,
the deprecated ``local_rank`` argument, transports reaching the layers through the converter, long training runs.

Reference behaviours covered: tests/modules/linear/test_linear.py:154-225 (sum backward), :227-305 (training),
:307-393 (column-only layout), :395-443 (bias init), :445-468 (parameter count), :470-502 (``local_rank``),
:504-584 (every transport), :586-675 (conversion keeps dtype, ``comm`` reaches the layers, unknown ``comm``).
"""

import warnings

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split

PATHS = {"weight_only": dict(input_grad=False, frozen=()), "input_only": dict(input_grad=True, frozen=("weight", "bias")),
         "both": dict(input_grad=True, frozen=())}


def _check_sum_backward(mesh, model_group, data_cut, param_cut, comm, path, tag):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.linear import LinearConfig

    torch.manual_seed(0)
    ref = torch.nn.Linear(8, 8).double()
    x = torch.randn(2, 4, 8, dtype=torch.float64)
    for name in PATHS[path]["frozen"]:
        getattr(ref, name).requires_grad_(False)
    xr = x.clone().requires_grad_(PATHS[path]["input_grad"])
    ref(xr).sum().backward()
    cfg = LinearConfig(model_group, device="cpu", comm=comm)
    layer = jb.modules.DistributedLinear(8, 8, "cpu", model_group, mesh["row"], mesh["col"], config=cfg, dtype=torch.float64)
    layer._load_global(ref.weight.data, ref.bias.data)
    for name in PATHS[path]["frozen"]:
        getattr(layer, name).requires_grad_(False)
    xl = split(x, data_cut).requires_grad_(PATHS[path]["input_grad"])
    y = layer(xl)
    assert_close(y, split(ref(x).detach(), data_cut), f"{tag}: output", 1e-12, 1e-12)
    y.sum().backward()                                             # the upstream gradient is an expanded scalar
    if PATHS[path]["input_grad"]:
        assert_close(xl.grad, split(xr.grad, data_cut), f"{tag}: dx", 1e-12, 1e-12)
    for name in ("weight", "bias"):
        g = getattr(layer, name).grad
        if name in PATHS[path]["frozen"]:
            assert g is None, f"{tag}: frozen {name} got a gradient"
        else:
            assert_close(g, split(getattr(ref, name).grad, param_cut[name]), f"{tag}: d{name}", 1e-12, 1e-12)


def _worker_sum_backward(rank, world, R, C):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": R, "col": C})
    row, col = mesh["row"], mesh["col"]
    for comm in ("isend", "batch_isend_irecv"):
        for path in PATHS:
            _check_sum_backward(mesh, mesh["model"], {1: row, 2: col}, {"weight": {0: row, 1: col}, "bias": {0: col}}, comm, path,
                                f"{R}x{C} {comm} {path}")
            if (R, C) == (2, 2):
                # the layout of attention's qkv / output projections: a column-only layer on four ranks,
                # tokens over the rows, features over the columns, weight replicated over the rows
                _check_sum_backward(mesh, col, {1: row, 2: col}, {"weight": {1: col}, "bias": {0: col}}, comm, path,
                                    f"column-only {comm} {path}")


@pytest.mark.parametrize("grid", [(1, 2), (2, 2), (4, 2)])
def test_summed_loss_on_every_gradient_path(grid):
    R, C = grid
    run_distributed(_worker_sum_backward, R * C, R, C, timeout=600)


def _worker_layouts(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist
    from jigsaw_b200 import convert

    M = jb.modules
    P = jb.parallel
    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col = mesh["row"], mesh["col"]
    col_mesh = {**mesh, "model": col}
    row_ranks = dist.get_process_group_ranks(row)
    ranks_of = lambda p: [dist.get_process_group_ranks(g) for g in P.replica_groups(p)]      # noqa: E731
    torch.manual_seed(0)
    serial = torch.nn.Linear(8, 8).double()
    # column-only: convert, merge, re-shard to row x col and back; the mark over the rows follows the layout
    layer = M.DistributedLinear.convert_to_jigsaw(serial, mesh, "cpu", model_kw="col")
    assert_close(layer.weight.data, split(serial.weight.data, {1: col}), "column-only: converted weight", 0, 0)
    assert_close(layer.bias.data, split(serial.bias.data, {0: col}), "column-only: converted bias", 0, 0)
    marked = ranks_of(layer.weight) == [row_ranks]

    def merged_equals(model_kw, what):
        w, b = layer.merge_weights(mesh, model_kw=model_kw)
        assert_close(w, serial.weight.data, f"{what}: merged weight", 0, 0)
        assert_close(b, serial.bias.data, f"{what}: merged bias", 0, 0)
        assert_close(layer.convert_to_torch(mesh, model_kw=model_kw).weight.data, serial.weight.data, f"{what}: converted back", 0, 0)

    merged_equals("col", "column-only")
    x = torch.randn(4, 4, 8, dtype=torch.float64)
    cuts = {1: row, 2: col}
    assert_close(layer(split(x, cuts)), split(serial(x).detach(), cuts), "column-only: output", 1e-12, 1e-12)
    layer.reshard_parameters(col_mesh, mesh)
    unmarked = ranks_of(layer.weight) == []
    merged_equals("model", "row x col after the re-shard")
    assert_close(layer(split(x, cuts)), split(serial(x).detach(), cuts), "row x col: output", 1e-12, 1e-12)
    layer.reshard_parameters(mesh, col_mesh)
    remarked = ranks_of(layer.weight) == [row_ranks]
    merged_equals("col", "column-only again")
    assert all_ok(marked and unmarked and remarked), "the weight's replica mark over the rows does not follow the layout"
    # bias initialisation: different seeds on every rank, yet the row replicas of the bias agree
    torch.manual_seed(mesh["model"].rank())
    fresh = M.DistributedLinear(6, 10, "cpu", mesh["model"], row, col)
    parts = [torch.empty_like(fresh.bias.data) for _ in range(4)]
    dist.all_gather(parts, fresh.bias.data, group=mesh["model"])
    assert torch.equal(parts[0], parts[2]) and torch.equal(parts[1], parts[3]) and not torch.equal(parts[0], parts[1])
    assert fresh.get_parameter_count() == 6 * 10 + 10                        # global, on every rank
    # the deprecated local_rank argument is accepted, warns and changes nothing
    torch.manual_seed(1)
    a = M.DistributedLinear(8, 8, "cpu", mesh["model"], row, col)
    torch.manual_seed(1)
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        b = M.DistributedLinear(8, 8, "cpu", mesh["model"], row, col, local_rank=3)
    assert any(issubclass(w.category, DeprecationWarning) for w in seen)
    assert torch.equal(a.weight, b.weight) and torch.equal(a.bias, b.bias)
    # conversion keeps the dtype both ways; comm= reaches every converted layer; an unknown transport is refused
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.GELU(), torch.nn.Linear(16, 8)).to(torch.bfloat16)
    conv = convert.convert_to_jigsaw(model, mesh, "cpu", comm="isend")
    assert all(p.dtype == torch.bfloat16 for p in conv.parameters())
    assert conv[0].convert_to_torch(mesh).weight.dtype == torch.bfloat16
    assert str(conv[0].config.comm) == "isend" and str(conv[2].config.comm) == "isend"
    with pytest.raises(ValueError):
        convert.convert_to_jigsaw(torch.nn.Linear(8, 8), mesh, "cpu", comm="carrier_pigeon")
    # many optimizer steps: the sharded layer follows the serial one, and its row replicas stay bit-identical
    torch.manual_seed(2)
    serial = torch.nn.Linear(8, 8).double()
    layer = M.DistributedLinear(8, 8, "cpu", mesh["model"], row, col, dtype=torch.float64)
    layer._load_global(serial.weight.data, serial.bias.data)
    opt_s, opt = torch.optim.SGD(serial.parameters(), lr=0.05, momentum=0.9), torch.optim.SGD(layer.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(3)
    for _ in range(25):
        xb = torch.randn(4, 6, 8, generator=g, dtype=torch.float64)
        opt_s.zero_grad()
        serial(xb).square().mean().backward()
        opt_s.step()
        opt.zero_grad()
        out = layer(split(xb, cuts))
        (out.square().sum() / xb[..., :1].numel() / 8).backward()       # the global mean, from local sums
        opt.step()
    w, b2 = layer.merge_weights(mesh)
    assert_close(w, serial.weight.data, "after 25 momentum steps: weight", 1e-10, 1e-10)
    assert_close(b2, serial.bias.data, "after 25 momentum steps: bias", 1e-10, 1e-10)
    jb.debug.assert_replica_consistency(layer, mesh)


def test_layouts_initialisation_conversion_and_training():
    run_distributed(_worker_layouts, 4, timeout=600)


def _worker_config_mismatch(rank, world):
    """A configuration object belongs to one kind of layer on one group size; a failed re-shard changes nothing
    (reference: tests/modules/linear/test_config_checks.py:113-170)."""
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.linear import LinearConfig

    m22, m14 = jb.make_process_mesh({"row": 2, "col": 2}), jb.make_process_mesh({"row": 1, "col": 4})
    M, model, row, col = jb.modules, m22["model"], m22["row"], m22["col"]
    refused = [
        lambda: M.DistributedLinear(8, 8, "cpu", model, row, col, config=LinearConfig(row, device="cpu")),
        lambda: M.DistributedLinear(8, 8, "cpu", model, row, col, config=LinearConfig(model, linear_layer=False, device="cpu")),
        lambda: M.DistributedMatMulXW("cpu", model, LinearConfig(model, device="cpu")),
        lambda: M.DistributedMatMulXTW("cpu", model, LinearConfig(row, linear_layer=False, device="cpu")),
    ]
    for build in refused:
        with pytest.raises(ValueError, match="different layer"):
            build()
    M.DistributedLinear(8, 8, "cpu", model, row, col, config=LinearConfig(model, device="cpu", comm="isend"))
    layer = M.DistributedLinear(6, 6, "cpu", model, row, col)
    weight, bias, config = layer.weight, layer.bias, layer.config
    with pytest.raises(ValueError, match="in_dim=6"):
        layer.reshard_parameters(m22, m14)                       # refused before anything is gathered
    assert layer.weight is weight and layer.bias is bias and layer.config is config and layer.model_group is model
    x = torch.randn(3, 3)
    assert tuple(layer(x).shape) == (3, 3)                        # and the layer still works on its old mesh
    assert all_ok(True)


def test_configurations_of_other_layers_and_failed_reshards():
    run_distributed(_worker_config_mismatch, 4, timeout=300)
