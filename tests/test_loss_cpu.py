"""Loss functionals and modules: torch parity without groups, ``vmap(grad)``, bf16 means, all seven module
wrappers on an eight-rank mesh (class axis and two reduce axes split), and training parity of a sharded linear
model against the undivided one under MSE and cross-entropy.

Reference behaviours covered: tests/modules/loss/test_loss.py:82-177 (no groups, vmap), :628-690 (bf16 means
accumulate in fp32), :735-836 (eight-way), :838-889 (module wrappers), :891-1060 (training parity).
"""

import pytest
import torch
import torch.nn.functional as F

from dist_utils import assert_close, run_distributed, split


def _fn():
    import jigsaw_b200 as jb

    return jb.modules.functional


def test_functionals_match_torch_without_groups():
    Fn = _fn()
    torch.manual_seed(0)
    logits = torch.randn(4, 7, 5, dtype=torch.float64, requires_grad=True)
    target = torch.randint(0, 7, (4, 5))
    for reduction in ("mean", "sum", "none"):
        assert torch.allclose(Fn.distributed_cross_entropy(logits, target, reduction=reduction),
                              F.cross_entropy(logits, target, reduction=reduction), atol=1e-12)
    logp = F.log_softmax(logits, dim=1)
    assert torch.allclose(Fn.distributed_nll_loss(logp, target), F.nll_loss(logp, target), atol=1e-12)
    probs = torch.rand(3, 6, dtype=torch.float64).clamp(0.02, 0.98)
    bt = torch.randint(0, 2, (3, 6)).double()
    raw = torch.randn(3, 6, dtype=torch.float64)
    assert torch.allclose(Fn.distributed_binary_cross_entropy(probs, bt), F.binary_cross_entropy(probs, bt), atol=1e-12)
    assert torch.allclose(Fn.distributed_binary_cross_entropy_with_logits(raw, bt), F.binary_cross_entropy_with_logits(raw, bt), atol=1e-12)
    pred, tgt = torch.randn(4, 7, 5, dtype=torch.float64), torch.randn(4, 7, 5, dtype=torch.float64)
    for reduction in ("mean", "sum", "none"):
        assert torch.allclose(Fn.distributed_mse_loss(pred, tgt, reduction=reduction), F.mse_loss(pred, tgt, reduction=reduction), atol=1e-12)
        assert torch.allclose(Fn.distributed_l1_loss(pred, tgt, reduction=reduction), F.l1_loss(pred, tgt, reduction=reduction), atol=1e-12)
        assert torch.allclose(Fn.distributed_smooth_l1_loss(pred, tgt, beta=0.7, reduction=reduction),
                              F.smooth_l1_loss(pred, tgt, beta=0.7, reduction=reduction), atol=1e-12)
    with pytest.raises(ValueError):
        Fn.distributed_mse_loss(pred, tgt, reduction="median")


@pytest.mark.parametrize("label_smoothing", [0.0, 0.1])
def test_vmap_of_grad_matches_a_loop(label_smoothing):
    from torch.func import grad, vmap

    Fn = _fn()
    e, n, c, s = 3, 4, 6, 5
    torch.manual_seed(1)
    logits = torch.randn(e, n, c, s, dtype=torch.float64)
    target = torch.randint(0, c, (e, n, s))

    def ce(lg, tg):
        return Fn.distributed_cross_entropy(lg, tg, reduction="mean", label_smoothing=label_smoothing)

    got = vmap(grad(ce))(logits, target)
    ref = torch.stack([grad(ce)(logits[i], target[i]) for i in range(e)])
    assert torch.allclose(got, ref, atol=1e-10)
    a, b = torch.randn(e, n, c, dtype=torch.float64), torch.randn(e, n, c, dtype=torch.float64)
    for loss in (Fn.distributed_mse_loss, Fn.distributed_l1_loss, Fn.distributed_smooth_l1_loss):
        got = vmap(grad(lambda p, q: loss(p, q, reduction="mean")))(a, b)
        ref = torch.stack([grad(lambda p, q: loss(p, q, reduction="mean"))(a[i], b[i]) for i in range(e)])
        assert torch.allclose(got, ref, atol=1e-10)


def test_half_precision_means_accumulate_in_fp32():
    """65536 bf16 elements of magnitude ~1: a bf16 running sum would stall at 256-ish; the mean must stay
    within bf16 rounding of the fp64 mean."""
    Fn = _fn()
    torch.manual_seed(2)
    a = (torch.rand(256, 256) + 0.5).bfloat16()
    b = torch.zeros(256, 256).bfloat16()
    for loss, ref in ((Fn.distributed_mse_loss, F.mse_loss), (Fn.distributed_l1_loss, F.l1_loss)):
        got = loss(a, b)
        want = ref(a.double(), b.double())
        assert abs(float(got) - float(want)) <= 1e-2 * float(want), (float(got), float(want))
    with torch.autocast("cpu", dtype=torch.bfloat16):
        got = Fn.distributed_mse_loss(a.float(), b.float())
    assert abs(float(got) - float(F.mse_loss(a.double(), b.double()))) <= 1e-2 * float(got)


def _worker_modules_eight_way(rank, world):
    """Class axis over ``col`` (2), the two remaining axes over ``sh`` (2) and ``sw`` (2): every module wrapper
    against torch on the undivided tensors, value and input gradient, accumulated over two micro-batches."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 2})
    sh, sw, col = mesh["sh"], mesh["sw"], mesh["col"]
    M = jb.modules
    g = torch.Generator().manual_seed(3)
    spec = {1: col, 2: sh, 3: sw}
    tspec = {1: sh, 2: sw}
    w = torch.rand(6, generator=g, dtype=torch.float64) + 0.5
    cases = [
        ("ce", M.DistributedCrossEntropyLoss(col, (sh, sw)), lambda a, t: F.cross_entropy(a, t), "index"),
        ("ce weight+smooth", M.DistributedCrossEntropyLoss(col, (sh, sw), weight=w, label_smoothing=0.2),
         lambda a, t: F.cross_entropy(a, t, weight=w, label_smoothing=0.2), "index"),
        ("ce sum", M.DistributedCrossEntropyLoss(col, (sh, sw), reduction="sum"), lambda a, t: F.cross_entropy(a, t, reduction="sum"), "index"),
        ("nll", M.DistributedNLLLoss(col, (sh, sw)), lambda a, t: F.nll_loss(a, t), "logp"),
        ("mse", M.DistributedMSELoss(reduce_groups=(sh, sw, col)), F.mse_loss, "dense"),
        ("l1", M.DistributedL1Loss(reduce_groups=(sh, sw, col)), F.l1_loss, "dense"),
        ("smooth_l1", M.DistributedSmoothL1Loss(beta=0.5, reduce_groups=(sh, sw, col)), lambda a, t: F.smooth_l1_loss(a, t, beta=0.5), "dense"),
        ("bce", M.DistributedBCELoss(reduce_groups=(sh, sw, col)), F.binary_cross_entropy, "prob"),
        ("bce logits", M.DistributedBCEWithLogitsLoss(reduce_groups=(sh, sw, col)), F.binary_cross_entropy_with_logits, "unit"),
    ]
    for name, module, ref_fn, kind in cases:
        assert module.get_parameter_count() == 0
        total = total_ref = 0.0
        xs_local, xs_ref = [], []
        for micro in range(2):
            a = torch.randn(2, 6, 4, 8, generator=g, dtype=torch.float64)
            if kind == "logp":
                a = torch.log_softmax(a, 1)
            if kind == "prob":
                a = torch.sigmoid(a)
            if kind in ("index", "logp"):
                t = torch.randint(0, 6, (2, 4, 8), generator=g)
                t[0, 0, micro] = -100
                tl = split(t, tspec)
            else:
                t = torch.rand(2, 6, 4, 8, generator=g, dtype=torch.float64)
                tl = split(t, spec)
            ar = a.clone().requires_grad_(True)
            al = split(a, spec).requires_grad_(True)
            total_ref = total_ref + ref_fn(ar, t)
            total = total + module(al, tl)
            xs_local.append(al)
            xs_ref.append(ar)
        assert_close(total, total_ref.detach(), f"{name}: value over two micro-batches", 1e-10, 1e-10)
        total.backward()
        total_ref.backward()
        for al, ar in zip(xs_local, xs_ref):
            assert_close(al.grad, split(ar.grad, spec), f"{name}: input gradient", 1e-10, 1e-10)


def test_module_wrappers_on_eight_ranks():
    run_distributed(_worker_modules_eight_way, 8, timeout=600)


def _worker_training_parity(rank, world):
    """A sharded linear classifier / regressor trained for a few SGD steps follows the undivided model:
    the loss values agree step by step and so do the final weights."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    for loss_name in ("mse", "ce"):
        torch.manual_seed(4)
        ref = torch.nn.Linear(8, 12).double()
        layer = jb.modules.DistributedLinear(8, 12, "cpu", model, row, col, dtype=torch.float64)
        layer._load_global(ref.weight.data, ref.bias.data)
        opt_ref = torch.optim.SGD(ref.parameters(), lr=0.1)
        opt = torch.optim.SGD(layer.parameters(), lr=0.1)
        if loss_name == "mse":
            loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(row, col))
        else:
            loss_fn = jb.modules.DistributedCrossEntropyLoss(col, (row,), dim=-1)
        g = torch.Generator().manual_seed(5)
        for step in range(5):
            x = torch.randn(4, 6, 8, generator=g, dtype=torch.float64)
            if loss_name == "mse":
                y = torch.randn(4, 6, 12, generator=g, dtype=torch.float64)
                want = F.mse_loss(ref(x), y)
                got = loss_fn(layer(split(x, {1: row, 2: col})), split(y, {1: row, 2: col}))
            else:
                y = torch.randint(0, 12, (4, 6), generator=g)
                want = F.cross_entropy(ref(x).flatten(0, 1), y.flatten())
                got = loss_fn(layer(split(x, {1: row, 2: col})), split(y, {1: row}))
            assert_close(got, want.detach(), f"{loss_name}: loss at step {step}", 1e-10, 1e-10)
            opt_ref.zero_grad()
            want.backward()
            opt_ref.step()
            opt.zero_grad()
            got.backward()
            opt.step()
        w, b = layer.merge_weights(mesh)
        assert_close(w, ref.weight.data, f"{loss_name}: trained weight", 1e-10, 1e-10)
        assert_close(b, ref.bias.data, f"{loss_name}: trained bias", 1e-10, 1e-10)


def test_training_parity_of_a_sharded_linear_model():
    run_distributed(_worker_training_parity, 4, timeout=300)
