"""Segmentation metrics over a sharded class dimension: arg-max (ties go to the lowest global index), confusion
matrices from logits and from class indices, ``ignore_index``, every derived metric against a straight
single-process computation, excluded and absent classes, the accumulating module, an eight-rank mesh.

Reference behaviours covered: tests/modules/metrics/test_segmentation.py:137-158 (arg-max), :160-245 (confusion
matrices), :247-343 (derived metrics), :345-382 (module accumulation), :384-405 (eight ranks).
"""

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split

C, N, H, W = 8, 2, 8, 8


def _ref_confusion(logits, target, ignore_index=None):
    pred = logits.argmax(1)
    keep = torch.ones_like(target, dtype=torch.bool) if ignore_index is None else target != ignore_index
    return torch.bincount(target[keep] * C + pred[keep], minlength=C * C).view(C, C)


def _ref_metrics(cm):
    cm = cm.double()
    tp, support, predicted = cm.diag(), cm.sum(1), cm.sum(0)
    union = support + predicted - tp
    present = union > 0
    nan = torch.full_like(tp, float("nan"))
    iou = torch.where(present, tp / union.clamp_min(1), nan)
    dice = torch.where(present, 2 * tp / (support + predicted).clamp_min(1), nan)
    precision = torch.where(predicted > 0, tp / predicted.clamp_min(1), nan)
    recall = torch.where(support > 0, tp / support.clamp_min(1), nan)
    total = cm.sum()
    pe = (support * predicted).sum() / total**2
    po = tp.sum() / total
    return {"per_class_iou": iou, "per_class_dice": dice, "per_class_precision": precision, "per_class_recall": recall,
            "mean_iou": iou.nanmean(), "mean_dice": dice.nanmean(), "pixel_accuracy": po, "mean_accuracy": recall.nanmean(),
            "frequency_weighted_iou": (torch.nan_to_num(iou) * support).sum() / total, "cohen_kappa": (po - pe) / (1 - pe)}


def _check_metrics(got, ref, tag):
    for key, want in ref.items():
        have = got[key].double()
        same_nan = torch.equal(torch.isnan(have), torch.isnan(want))
        assert all_ok(same_nan), f"{tag}: {key} marks other classes as absent"
        assert_close(torch.nan_to_num(have), torch.nan_to_num(want), f"{tag}: {key}", 1e-9, 1e-12)


def _worker_metrics(rank, world, axes):
    import jigsaw_b200 as jb

    Fn = jb.modules.functional
    mesh = jb.make_process_mesh(dict(axes), model_parallel_axes=("row", "col"))
    row, col = mesh["row"], mesh["col"]
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(N, C, H, W, generator=g, dtype=torch.float64)
    logits[0, 2, 0, 0] = logits[0, 4, 0, 0] = 50.0                     # a tie between classes of different shards
    target = torch.randint(0, C, (N, H, W), generator=g)
    lcut, tcut = {1: col, 2: row}, {1: row}
    tag = str(dict(axes))
    # arg-max
    got = Fn.distributed_argmax(split(logits, lcut), dim=1, group=col)
    assert all_ok(torch.equal(got, split(logits.argmax(1), tcut))), f"{tag}: arg-max"
    assert int(split(logits.argmax(1), tcut)[0, 0, 0]) == 2 if row.rank() == 0 else True
    # confusion matrices
    kw = dict(channel_group=col, reduce_groups=(row,))
    cm = Fn.distributed_confusion_matrix(split(logits, lcut), split(target, tcut), C, **kw)
    assert all_ok(torch.equal(cm, _ref_confusion(logits, target)) and int(cm.sum()) == N * H * W and cm.dtype == torch.int64), f"{tag}: confusion"
    void = target.clone()
    void[:, ::3, :] = 255
    cm_void = Fn.distributed_confusion_matrix(split(logits, lcut), split(void, tcut), C, ignore_index=255, **kw)
    assert all_ok(torch.equal(cm_void, _ref_confusion(logits, void, 255)) and int(cm_void.sum()) == int((void != 255).sum())), f"{tag}: ignore_index"
    cm_idx = Fn.distributed_confusion_matrix(split(logits.argmax(1), tcut), split(target, tcut), C, reduce_groups=(row,))
    assert all_ok(torch.equal(cm_idx, cm)), f"{tag}: confusion from class indices"
    if col.size() > 1:
        with pytest.raises(ValueError, match="num_classes"):
            Fn.distributed_confusion_matrix(split(logits, lcut), split(target, tcut), C + 1, **kw)
    # derived metrics, excluded classes, a class that never occurs
    _check_metrics(Fn.confusion_to_metrics(cm), _ref_metrics(_ref_confusion(logits, target)), tag)
    excl = _ref_confusion(logits, target).clone()
    excl[[0, 3], :] = 0
    excl[:, [0, 3]] = 0
    got = Fn.confusion_to_metrics(cm, exclude=[0, 3])
    _check_metrics(got, _ref_metrics(excl), f"{tag}: exclude")
    assert bool(torch.isnan(got["per_class_iou"][0]) and torch.isnan(got["per_class_iou"][3]))
    lonely_t, lonely_l = target.clone(), logits.clone()
    lonely_t[lonely_t == 0] = 1
    lonely_l[:, 0] = -1e4
    got = Fn.confusion_to_metrics(Fn.distributed_confusion_matrix(split(lonely_l, lcut), split(lonely_t, tcut), C, **kw))
    assert bool(torch.isnan(got["per_class_iou"][0])) and not bool(torch.isnan(got["mean_iou"]))
    _check_metrics(got, _ref_metrics(_ref_confusion(lonely_l, lonely_t)), f"{tag}: absent class")
    # the module accumulates over batches; reset starts over; forward returns the batch's matrix
    metric = jb.modules.DistributedSegmentationMetrics(C, col, (row,), ignore_index=255)
    total = torch.zeros(C, C, dtype=torch.int64)
    for seed in (1, 2, 3):
        gg = torch.Generator().manual_seed(seed)
        lg = torch.randn(N, C, H, W, generator=gg, dtype=torch.float64)
        tg = torch.randint(0, C, (N, H, W), generator=gg)
        tg[:, 0, :] = 255
        metric.update(split(lg, lcut), split(tg, tcut))
        total += _ref_confusion(lg, tg, 255)
    res = metric.compute()
    assert all_ok(torch.equal(res["confusion"], total)), f"{tag}: accumulated confusion"
    _check_metrics(res, _ref_metrics(total), f"{tag}: accumulated metrics")
    metric.reset()
    assert int(metric.compute()["confusion"].sum()) == 0


@pytest.mark.parametrize("axes", [(("row", 2), ("col", 2)), (("row", 1), ("col", 4)), (("row", 4), ("col", 1)),
                                  (("dp", 2), ("row", 1), ("col", 2))], ids=["2x2", "1x4", "4x1", "2x1x2"])
def test_metrics_on_four_ranks(axes):
    run_distributed(_worker_metrics, 4, axes, timeout=300)


def test_metrics_on_eight_ranks():
    run_distributed(_worker_metrics, 8, (("row", 4), ("col", 2)), timeout=300)


def test_single_process_paths():
    """No group at all: logits recognised by their extra axis, the explicit switch either way, a module without
    parameters whose running matrix adds up over calls (reference: tests/modules/metrics/test_segmentation_local.py)."""
    from jigsaw_b200.modules.metrics import DistributedSegmentationMetrics, distributed_confusion_matrix

    gen = torch.Generator().manual_seed(0)
    logits = torch.randn(N, C, 5, 3, generator=gen)
    target = torch.randint(0, C, (N, 5, 3), generator=gen)
    want = _ref_confusion(logits, target)
    assert torch.equal(distributed_confusion_matrix(logits, target, C), want)
    assert torch.equal(distributed_confusion_matrix(logits, target, C, pred_is_logits=True), want)
    assert torch.equal(distributed_confusion_matrix(logits.argmax(1), target, C, pred_is_logits=False), want)
    assert torch.equal(distributed_confusion_matrix(logits.argmax(1), target, C), want)               # indices: same rank as the target
    moved = logits.movedim(1, -1)                                                                       # classes last
    assert torch.equal(distributed_confusion_matrix(moved, target, C, dim=-1), want)
    metric = DistributedSegmentationMetrics(C)
    assert metric.get_parameter_count() == 0 and not list(metric.parameters()) and not metric.state_dict()
    metric(logits, target)
    metric.update(logits, target)
    assert torch.equal(metric.confusion, 2 * want)
    assert abs(float(metric.compute()["pixel_accuracy"]) - float(_ref_metrics(want)["pixel_accuracy"])) < 1e-12
    metric.reset()
    assert int(metric.confusion.sum()) == 0


def _worker_one_group_for_a_sequence(rank, world):
    import torch.distributed as dist
    from jigsaw_b200.modules.metrics import distributed_confusion_matrix

    gen = torch.Generator().manual_seed(0)
    logits, target = torch.randn(N, C, 5, 3, generator=gen), torch.randint(0, C, (N, 5, 3), generator=gen)
    got = distributed_confusion_matrix(logits, target, C, reduce_groups=dist.group.WORLD)               # a group, not a list of groups
    assert torch.equal(got, world * _ref_confusion(logits, target))                                    # every rank held the same data


def test_a_single_group_where_a_sequence_is_expected():
    run_distributed(_worker_one_group_for_a_sequence, 2)
