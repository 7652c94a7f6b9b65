"""Layer parity on CPU/gloo ranks: every distributed layer against its torch counterpart on
the gathered tensors (output, input gradient, parameter gradients)."""

import pytest
import torch
import torch.nn.functional as F

from dist_utils import assert_close, run_distributed, split


def _mesh_rc():
    import jigsaw_b200 as jb

    return jb.make_process_mesh({"row": 2, "col": 2})


def _worker_linear(rank, world):
    import jigsaw_b200 as jb

    mesh = _mesh_rc()
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    torch.manual_seed(0)
    ref = torch.nn.Linear(8, 12).double()
    x = torch.randn(3, 6, 8, dtype=torch.float64)
    xr = x.clone().requires_grad_(True)
    yr = ref(xr)
    gy = torch.randn_like(yr)
    yr.backward(gy)
    for mg in (model, col):     # 2x2 block layout, and projection layout (weight replicated over rows)
        layer = jb.modules.DistributedLinear(8, 12, "cpu", mg, row, col, dtype=torch.float64)
        layer._load_global(ref.weight.data, ref.bias.data)
        spec = {1: row, 2: col}
        xl = split(x, spec).requires_grad_(True)
        y = layer(xl)
        assert_close(y, split(yr.detach(), spec), "linear out", 1e-10, 1e-10)
        y.backward(split(gy, spec))
        assert_close(xl.grad, split(xr.grad, spec), "linear dx", 1e-10, 1e-10)
        wspec = {0: row, 1: col} if mg is model else {1: col}
        assert_close(layer.weight.grad, split(ref.weight.grad, wspec), "linear dW", 1e-10, 1e-10)
        assert_close(layer.bias.grad, split(ref.bias.grad, {0: col}), "linear db", 1e-10, 1e-10)
        back = layer.convert_to_torch(mesh)
        assert_close(back.weight.data, ref.weight.data, "linear merge", 0, 0)
        assert layer.get_parameter_count() == 8 * 12 + 12
    # converter + init statistics: fans come from the global shape
    torch.manual_seed(1)
    conv = jb.modules.DistributedLinear.convert_to_jigsaw(torch.nn.Linear(8, 12), mesh, "cpu")
    assert conv.weight.shape == (6, 4) and conv.bias.shape == (6,)
    big = jb.modules.DistributedLinear(512, 512, "cpu", model, row, col)
    bound = 1.0 / 512 ** 0.5
    assert big.weight.abs().max() <= bound + 1e-6 and big.weight.abs().max() > 0.9 * bound
    # matmul modules on the bare model group
    A = torch.randn(2, 8, 6, dtype=torch.float64)
    B = torch.randn(2, 10, 6, dtype=torch.float64)
    mm = jb.modules.DistributedMatMulXWT("cpu", model)
    out = mm(split(A, {1: row, 2: col}), split(B, {1: row, 2: col}))
    assert_close(out, split(A @ B.transpose(-1, -2), {1: row, 2: col}), "XWT", 1e-10, 1e-10)
    Bw = torch.randn(2, 6, 10, dtype=torch.float64)
    out = jb.modules.DistributedMatMulXW("cpu", model)(split(A, {1: row, 2: col}), split(Bw, {1: row, 2: col}))
    assert_close(out, split(A @ Bw, {1: row, 2: col}), "XW", 1e-10, 1e-10)
    At = torch.randn(2, 6, 8, dtype=torch.float64)
    out = jb.modules.DistributedMatMulXTW("cpu", model)(split(At, {1: row, 2: col}), split(Bw, {1: row, 2: col}))
    assert_close(out, split(At.transpose(-1, -2) @ Bw, {1: row, 2: col}), "XTW", 1e-10, 1e-10)


def _worker_norms(rank, world):
    import jigsaw_b200 as jb

    mesh = _mesh_rc()
    row, col = mesh["row"], mesh["col"]
    torch.manual_seed(0)
    ref = torch.nn.LayerNorm(16).double()
    ref.weight.data.uniform_(0.5, 1.5)
    ref.bias.data.uniform_(-0.5, 0.5)
    x = torch.randn(2, 6, 16, dtype=torch.float64)
    xr = x.clone().requires_grad_(True)
    yr = ref(xr)
    gy = torch.randn_like(yr)
    yr.backward(gy)
    ln = jb.modules.DistributedLayerNorm.convert_to_jigsaw(ref, mesh, "cpu")
    spec = {1: row, 2: col}
    xl = split(x, spec).requires_grad_(True)
    y = ln(xl)
    assert_close(y, split(yr.detach(), spec), "ln out", 1e-10, 1e-10)
    y.backward(split(gy, spec))
    assert_close(xl.grad, split(xr.grad, spec), "ln dx", 1e-10, 1e-10)
    assert_close(ln.weight.grad, split(ref.weight.grad, {0: col}), "ln dW", 1e-10, 1e-10)
    assert_close(ln.bias.grad, split(ref.bias.grad, {0: col}), "ln db", 1e-10, 1e-10)
    assert_close(ln.convert_to_torch(mesh).weight.data, ref.weight.data, "ln merge", 0, 0)
    # group norm: channels over col, spatial (last axis) over row
    gref = torch.nn.GroupNorm(4, 8).double()
    gref.weight.data.uniform_(0.5, 1.5)
    gref.bias.data.uniform_(-0.5, 0.5)
    x = torch.randn(2, 8, 6, 10, dtype=torch.float64)
    xr = x.clone().requires_grad_(True)
    yr = gref(xr)
    gy = torch.randn_like(yr)
    yr.backward(gy)
    gn = jb.modules.DistributedGroupNorm.convert_to_jigsaw(gref, mesh, "cpu")
    spec = {1: col, 3: row}
    xl = split(x, spec).requires_grad_(True)
    y = gn(xl)
    assert_close(y, split(yr.detach(), spec), "gn out", 1e-10, 1e-10)
    y.backward(split(gy, spec))
    assert_close(xl.grad, split(xr.grad, spec), "gn dx", 1e-10, 1e-10)
    assert_close(gn.weight.grad, split(gref.weight.grad, {0: col}), "gn dW", 1e-10, 1e-10)
    # softmax family over a sharded dim
    x = torch.randn(3, 5, 12, dtype=torch.float64)
    xr = x.clone().requires_grad_(True)
    yr = torch.softmax(xr, -1)
    gy = torch.randn_like(yr)
    yr.backward(gy)
    xl = split(x, {2: col}).requires_grad_(True)
    y = jb.modules.DistributedSoftmax(col, -1)(xl)
    assert_close(y, split(yr.detach(), {2: col}), "softmax", 1e-12, 1e-12)
    y.backward(split(gy, {2: col}))
    assert_close(xl.grad, split(xr.grad, {2: col}), "softmax dx", 1e-12, 1e-12)
    ls = jb.modules.functional.distributed_log_softmax(split(x, {2: col}), -1, col)
    assert_close(ls, split(torch.log_softmax(x, -1), {2: col}), "log_softmax", 1e-12, 1e-12)
    xt = x.clone()
    xt[0, 0, 3] = xt[0, 0, 9] = 100.0          # tie across shards -> lowest global index
    am = jb.modules.functional.distributed_argmax(split(xt, {2: col}), 2, col)
    assert_close(am, xt.argmax(-1), "argmax", 0, 0)
    assert int(am[0, 0]) == 3


def _worker_losses(rank, world):
    import jigsaw_b200 as jb

    mesh = _mesh_rc()
    row, col = mesh["row"], mesh["col"]
    Fn = jb.modules.functional
    torch.manual_seed(0)
    logits = torch.randn(4, 6, 10, dtype=torch.float64)
    target = torch.randint(0, 6, (4, 10))
    target[0, 0] = -100
    w = torch.rand(6, dtype=torch.float64) + 0.5
    spec = {1: col, 2: row}
    for kw in (dict(), dict(weight=w), dict(label_smoothing=0.1), dict(reduction="sum"), dict(reduction="none")):
        lr = logits.clone().requires_grad_(True)
        ref = F.cross_entropy(lr, target, **kw)
        ll = split(logits, spec).requires_grad_(True)
        out = Fn.distributed_cross_entropy(ll, split(target, {1: row}), channel_group=col, reduce_groups=(row,), **kw)
        if kw.get("reduction") == "none":
            assert_close(out, split(ref.detach(), {1: row}), f"ce none", 1e-10, 1e-10)
            continue
        assert_close(out, ref.detach(), f"ce {kw}", 1e-10, 1e-10)
        ref.backward()
        out.backward()
        assert_close(ll.grad, split(lr.grad, spec), f"ce grad {kw}", 1e-10, 1e-10)
    probs = torch.softmax(torch.randn(4, 6, 10, dtype=torch.float64), 1)
    out = Fn.distributed_cross_entropy(split(logits, spec), split(probs, spec), channel_group=col, reduce_groups=(row,))
    assert_close(out, F.cross_entropy(logits, probs), "ce prob", 1e-10, 1e-10)
    with pytest.raises(NotImplementedError):
        Fn.distributed_cross_entropy(split(logits, spec), split(probs, spec), channel_group=col, label_smoothing=0.1)
    logp = torch.log_softmax(logits, 1)
    out = Fn.distributed_nll_loss(split(logp, spec), split(target, {1: row}), weight=w, channel_group=col, reduce_groups=(row,))
    assert_close(out, F.nll_loss(logp, target, weight=w), "nll", 1e-10, 1e-10)
    # elementwise losses: every sharding group goes into reduce_groups
    a = torch.randn(4, 6, 10, dtype=torch.float64)
    b = torch.randn(4, 6, 10, dtype=torch.float64)
    for name, fn, ref_fn, kw in [
        ("mse", Fn.distributed_mse_loss, F.mse_loss, {}),
        ("l1", Fn.distributed_l1_loss, F.l1_loss, {}),
        ("huber", Fn.distributed_smooth_l1_loss, F.smooth_l1_loss, {"beta": 0.7}),
    ]:
        for red in ("mean", "sum"):
            ar = a.clone().requires_grad_(True)
            ref = ref_fn(ar, b, reduction=red, **kw)
            al = split(a, spec).requires_grad_(True)
            out = fn(al, split(b, spec), reduction=red, reduce_groups=(row, col), **kw)
            assert_close(out, ref.detach(), f"{name} {red}", 1e-10, 1e-10)
            ref.backward()
            out.backward()
            assert_close(al.grad, split(ar.grad, spec), f"{name} grad {red}", 1e-10, 1e-10)
    t01 = torch.rand(4, 6, 10, dtype=torch.float64)
    pw = torch.rand(10, dtype=torch.float64) + 0.5
    out = Fn.distributed_binary_cross_entropy_with_logits(split(a, spec), split(t01, spec), pos_weight=split(pw, {0: row}),
                                                          reduce_groups=(row, col))
    assert_close(out, F.binary_cross_entropy_with_logits(a, t01, pos_weight=pw), "bce logits", 1e-10, 1e-10)
    out = Fn.distributed_binary_cross_entropy(split(torch.sigmoid(a), spec), split(t01, spec), reduce_groups=(row, col))
    assert_close(out, F.binary_cross_entropy(torch.sigmoid(a), t01), "bce", 1e-10, 1e-10)
    # modules and the metrics accumulator
    m = jb.modules.DistributedCrossEntropyLoss(col, (row,), label_smoothing=0.1)
    assert_close(m(split(logits, spec), split(target, {1: row})), F.cross_entropy(logits, target, label_smoothing=0.1), "ce module", 1e-10, 1e-10)
    assert m.get_parameter_count() == 0
    metric = jb.modules.DistributedSegmentationMetrics(6, col, (row,), ignore_index=-100)
    metric.update(split(logits, spec), split(target, {1: row}))
    res = metric.compute()
    pred = logits.argmax(1)
    keep = target != -100
    cm = torch.bincount(target[keep] * 6 + pred[keep], minlength=36).view(6, 6)
    assert_close(res["confusion"], cm, "confusion", 0, 0)
    acc = (pred[keep] == target[keep]).double().mean()
    assert_close(res["pixel_accuracy"], acc, "pixel accuracy", 1e-12, 1e-12)
    red = Fn.redundant_all_reduce(torch.ones(2), (row, col))
    assert_close(red, torch.full((2,), 4.0), "redundant_all_reduce", 0, 0)


def _worker_roll_permute(rank, world):
    import jigsaw_b200 as jb

    mesh = _mesh_rc()
    row, col = mesh["row"], mesh["col"]
    torch.manual_seed(0)
    x = torch.randn(2, 8, 12, 3, dtype=torch.float64)
    spec = {1: row, 2: col}
    for shifts in [(3, -2), (0, 5), (-7, 11), (4, 6), (9, 1)]:
        ref_in = x.clone().requires_grad_(True)
        ref = torch.roll(ref_in, shifts, (1, 2))
        gy = torch.randn_like(ref)
        ref.backward(gy)
        layer = jb.modules.DistributedRoll(shifts, (1, 2), (1, 2), (row, col), "cpu")
        xl = split(x, spec).requires_grad_(True)
        y = layer(xl)
        assert_close(y, split(ref.detach(), spec), f"roll {shifts}", 0, 0)
        y.backward(split(gy, spec))
        assert_close(xl.grad, split(ref_in.grad, spec), f"roll grad {shifts}", 0, 0)
    conv = jb.modules.DistributedRoll.convert_to_jigsaw(jb.modules.Roll((2,), (-2,)), mesh, "cpu")
    assert conv.distributed_dims == (-2,) and conv.get_parameter_count() == 0
    # permute with a swap of the sharded axes
    t = torch.randn(3, 8, 12, dtype=torch.float64)
    out = jb.modules.functional.distributed_permute(split(t, {1: row, 2: col}), (0, 2, 1), 1, 2, None, "cpu", mesh)
    assert_close(out, split(t.permute(0, 2, 1), {1: row, 2: col}), "permute swap", 0, 0)
    out = jb.modules.functional.distributed_permute(split(t, {1: row, 2: col}), (0, 1, 2), 1, 2, None, "cpu", mesh)
    assert_close(out, split(t, {1: row, 2: col}), "permute id", 0, 0)
    with pytest.raises(ValueError):
        jb.modules.functional.distributed_permute(split(t, {1: row, 2: col}), (1, 0, 2), 1, 2, None, "cpu", mesh)


def test_linear_and_matmul():
    run_distributed(_worker_linear, 4)


def test_norms_and_softmax():
    run_distributed(_worker_norms, 4)


def test_losses_and_metrics():
    run_distributed(_worker_losses, 4)


def test_roll_and_permute():
    run_distributed(_worker_roll_permute, 4)
