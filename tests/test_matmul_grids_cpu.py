"""2-D block matrix products on CPU/gloo ranks: every kind (XWT, XW, XTW) on every grid the reference
implements (1x2, 2x2, 4x2) over every CPU transport, forward and both operand gradients against the dense
product of the gathered operands; frozen operands (their collectives are skipped consistently);
``DistributedLinear`` on grids the reference does not have (3x2, 2x3, 1x4).

Reference behaviours covered: tests/modules/linear/test_matmul_nway.py:96-185 (kinds x grids x transports,
reconstruction with gather_results), tests/modules/linear/test_grad_skip.py (frozen operands)."""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split

GRIDS = {2: (1, 2), 4: (2, 2), 8: (4, 2)}


def _dense(kind, X, W):
    if kind == "xwt":
        return X @ W.transpose(-1, -2)
    if kind == "xw":
        return X @ W
    return X.transpose(-1, -2) @ W


def _worker_matmul_kinds(rank, world, comm, kind):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.linear import LinearConfig

    R, C = GRIDS[world]
    mesh = jb.make_process_mesh({"row": R, "col": C})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    cut = {1: row, 2: col}
    torch.manual_seed(0)
    M, K, N = 8 * R * C, 4 * R * C, 2 * R * C            # every dimension divides by R, C and R * C
    shapes = {"xwt": ((2, M, K), (2, N, K)), "xw": ((2, M, K), (2, K, N)), "xtw": ((2, K, M), (2, K, N))}
    classes = {"xwt": jb.modules.DistributedMatMulXWT, "xw": jb.modules.DistributedMatMulXW, "xtw": jb.modules.DistributedMatMulXTW}
    for kind, (sx, sw) in ((kind, shapes[kind]),):
        for frozen in (None, "x", "w"):
            X = torch.randn(*sx, dtype=torch.float64)
            W = torch.randn(*sw, dtype=torch.float64)
            Xr, Wr = X.clone().requires_grad_(frozen != "x"), W.clone().requires_grad_(frozen != "w")
            Yr = _dense(kind, Xr, Wr)
            G = torch.randn_like(Yr)
            Yr.backward(G)
            layer = classes[kind]("cpu", model, LinearConfig(model, linear_layer=False, device="cpu", comm=comm))
            xl = split(X, cut).requires_grad_(frozen != "x")
            wl = split(W, cut).requires_grad_(frozen != "w")
            y = layer(xl, wl)
            assert_close(y, split(Yr.detach(), cut), f"{kind} {comm} frozen={frozen}: product", 1e-10, 1e-10)
            y.backward(split(G, cut))
            if frozen != "x":
                assert_close(xl.grad, split(Xr.grad, cut), f"{kind} {comm} frozen={frozen}: dX", 1e-10, 1e-10)
            else:
                assert xl.grad is None
            if frozen != "w":
                assert_close(wl.grad, split(Wr.grad, cut), f"{kind} {comm} frozen={frozen}: dW", 1e-10, 1e-10)
            else:
                assert wl.grad is None


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("comm", ["batch_isend_irecv", "isend"])
@pytest.mark.parametrize("kind", ["xwt", "xw", "xtw"])
def test_matmul_kinds_on_reference_grids(kind, world, comm):
    run_distributed(_worker_matmul_kinds, world, comm, kind, timeout=300)


def _worker_linear_any_grid(rank, world, R, C):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": R, "col": C})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    torch.manual_seed(1)
    fin, fout = 2 * R * C, 3 * R * C
    ref = torch.nn.Linear(fin, fout).double()
    x = torch.randn(2, 2 * R, fin, dtype=torch.float64)
    cut = {1: row, 2: col}
    for frozen_weight in (False, True):
        ref.zero_grad()
        ref.weight.requires_grad_(not frozen_weight)
        xr = x.clone().requires_grad_(True)
        yr = ref(xr)
        g = torch.randn_like(yr)
        yr.backward(g)
        layer = jb.modules.DistributedLinear(fin, fout, "cpu", model, row, col, dtype=torch.float64)
        layer._load_global(ref.weight.data, ref.bias.data)
        layer.weight.requires_grad_(not frozen_weight)
        xl = split(x, cut).requires_grad_(True)
        y = layer(xl)
        assert_close(y, split(yr.detach(), cut), f"{R}x{C}: output", 1e-10, 1e-10)
        y.backward(split(g, cut))
        assert_close(xl.grad, split(xr.grad, cut), f"{R}x{C}: dx", 1e-10, 1e-10)
        if frozen_weight:
            assert layer.weight.grad is None
        else:
            assert_close(layer.weight.grad, split(ref.weight.grad, {0: row, 1: col}), f"{R}x{C}: dW", 1e-10, 1e-10)
        assert_close(layer.bias.grad, split(ref.bias.grad, {0: col}), f"{R}x{C}: db", 1e-10, 1e-10)


@pytest.mark.parametrize("grid", [(3, 2), (2, 3), (1, 4), (4, 1)])
def test_linear_on_grids_beyond_the_reference(grid):
    R, C = grid
    run_distributed(_worker_linear_any_grid, R * C, R, C, timeout=300)
