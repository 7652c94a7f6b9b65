"""``clip_grad_norm_`` on sharded and replicated parameters: every element of the undivided model counts once.

Reference behaviours covered: tests/test_clip.py:64-82 (replicas clip like torch on one rank), :84-101 (shards and
replicas counted once), :103-112 (no clipping below the bound), :114-129 (a rank without gradients), :131-142
(replica group outside the clipping group), :144-148 (non-finite norm), :150-169 (half precision does not
overflow), :171-186 (dtype promotion over all parameters), :203-235 (a converted model against the serial one).
"""

import copy
import math

import pytest
import torch

from dist_utils import assert_close, run_distributed, split

NORMS = (2.0, 1.0, 3.0, math.inf)


def _with_grad(t):
    p = torch.nn.Parameter(torch.zeros_like(t))
    p.grad = t.clone()
    return p


def _worker_clip(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist

    P = jb.parallel
    mesh = jb.make_process_mesh({"a": 2, "b": 2}, model_parallel_axes=("a", "b"))
    a, b, model = mesh["a"], mesh["b"], mesh["model"]
    world_group = dist.group.WORLD
    # 1. parameters replicated over the whole group clip like torch on one rank
    for norm in NORMS:
        g = torch.Generator().manual_seed(0)
        grads = [torch.randn(5, 3, generator=g), torch.randn(7, generator=g)]
        ours, ref = [_with_grad(x) for x in grads], [_with_grad(x) for x in grads]
        for p in ours:
            P.mark_replicated(p, world_group)
        total = P.clip_grad_norm_(ours, 0.5, world_group, norm)
        want = torch.nn.utils.clip_grad_norm_(ref, 0.5, norm)
        assert_close(total, want, f"replicas: norm {norm}", 1e-5, 1e-6)
        for p, q in zip(ours, ref):
            assert_close(p.grad, q.grad, f"replicas: gradients {norm}", 1e-5, 1e-7)
    # 2. a sharded parameter (own values per rank), one replicated over `a`, one replicated over everything
    for norm in NORMS:
        sharded = _with_grad(torch.full((3,), float(rank + 1), dtype=torch.float64))
        rep_a = _with_grad(torch.full((2,), float(b.rank() + 2), dtype=torch.float64))
        rep_all = _with_grad(torch.full((1,), 5.0, dtype=torch.float64))
        P.mark_replicated(rep_a, a)
        P.mark_replicated(rep_all, [a, b])
        if math.isinf(norm):
            want = 5.0
        else:
            want = (sum(3 * float(r + 1) ** norm for r in range(4)) + sum(2 * float(j + 2) ** norm for j in range(2)) + 5.0**norm) ** (1 / norm)
        params = [sharded, rep_a, rep_all]
        before = [p.grad.clone() for p in params]
        total = P.clip_grad_norm_(params, want / 2, model, norm)
        assert total.dtype == torch.float64
        assert_close(total, torch.tensor(want, dtype=torch.float64), f"mixed: norm {norm}", 1e-12, 0)
        coef = (want / 2) / (want + 1e-6)
        for p, g0 in zip(params, before):
            assert_close(p.grad, g0 * coef, f"mixed: gradients {norm}", 1e-12, 1e-14)
        # below the bound nothing changes
        before = [p.grad.clone() for p in params]
        P.clip_grad_norm_(params, 10 * want, model, norm)
        for p, g0 in zip(params, before):
            assert_close(p.grad, g0, f"mixed: untouched below the bound {norm}", 0, 0)
    # 3. a rank without gradients still joins and gets the norm
    p = torch.nn.Parameter(torch.zeros(2))
    if rank != 0:
        p.grad = torch.full((2,), 3.0)
    total = P.clip_grad_norm_([p], 1.0, world_group)
    assert_close(total, torch.tensor(math.sqrt(18 * 3)), "rank without gradients", 1e-6, 0)
    # 4. a replica group that is not inside the clipping group: every rank raises, also the one without a gradient
    for norm in (2.0, math.inf):
        p = torch.nn.Parameter(torch.ones(2))
        if rank != 0:
            p.grad = torch.ones_like(p)
        P.mark_replicated(p, a)
        with pytest.raises(ValueError, match="model-parallel group"):
            P.clip_grad_norm_([p], 1.0, b, norm)
    # 5. non-finite norm
    with pytest.raises(RuntimeError, match="non-finite"):
        P.clip_grad_norm_([_with_grad(torch.tensor([1.0, math.inf]))], 1.0, world_group, error_if_nonfinite=True)
    # 6. a float16 gradient whose norm (1e5) exceeds float16's range still clips; the norm comes back in float32
    p = _with_grad(torch.full((10000,), 1000.0, dtype=torch.float16))
    P.mark_replicated(p, world_group)
    total = P.clip_grad_norm_([p], 1.0, world_group)
    assert total.dtype == torch.float32
    assert_close(total, torch.tensor(1e5), "half precision: norm", 1e-5, 0)
    assert_close(p.grad, torch.full_like(p.grad, 0.01), "half precision: clipped gradient", 1e-3, 0)
    # 7. the norm's dtype comes from every parameter, also those without gradients on this rank
    half = _with_grad(torch.ones(4, dtype=torch.bfloat16))
    wide = torch.nn.Parameter(torch.ones(2, dtype=torch.float64))
    if rank != 0:
        wide.grad = torch.ones_like(wide)
    for q in (half, wide):
        P.mark_replicated(q, world_group)
    assert P.clip_grad_norm_([half, wide], 100.0, world_group).dtype == torch.float64


def test_clipping_counts_every_element_once():
    run_distributed(_worker_clip, 4, timeout=300)


def _worker_converted_model(rank, world):
    """A converted MLP + convolution model clips like the serial one: same total norm, same gradients."""
    import jigsaw_b200 as jb
    from jigsaw_b200 import convert

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col = mesh["row"], mesh["col"]
    torch.manual_seed(3)
    serial = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.GELU(), torch.nn.LayerNorm(16), torch.nn.Linear(16, 8)).double()
    dist_model = convert.convert_to_jigsaw(copy.deepcopy(serial), mesh, "cpu")
    x = torch.randn(2, 6, 8, dtype=torch.float64)
    for norm in (2.0, math.inf):
        serial.zero_grad()
        dist_model.zero_grad()
        serial(x).square().sum().backward()
        dist_model(split(x, {1: row, 2: col})).square().sum().backward()
        want = torch.nn.utils.clip_grad_norm_(serial.parameters(), 0.1, norm)
        total = jb.parallel.clip_grad_norm_(dist_model.parameters(), 0.1, mesh["model"], norm)
        assert_close(total, want, f"converted model: norm {norm}", 1e-10, 1e-12)
        for i in (0, 3):
            assert_close(dist_model[i].weight.grad, split(serial[i].weight.grad, {0: row, 1: col}),
                         f"converted model: clipped weight gradient of layer {i}, norm {norm}", 1e-10, 1e-12)
            assert_close(dist_model[i].bias.grad, split(serial[i].bias.grad, {0: col}),
                         f"converted model: clipped bias gradient of layer {i}, norm {norm}", 1e-10, 1e-12)


def test_converted_model_clips_like_the_serial_one():
    run_distributed(_worker_converted_model, 4, timeout=300)
