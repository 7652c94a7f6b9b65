"""Replica marks, in-graph gradient sync, DDP composition (both modes), clipping, debug checks."""

import os

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split


def _tiny_model(mesh, seed=0):
    import jigsaw_b200 as jb

    torch.manual_seed(seed)
    M = jb.modules
    return torch.nn.Sequential(
        M.DistributedConv2d(2, 4, 3, "cpu", (mesh["sh"], mesh["sw"]), mesh["col"], padding=1),
        torch.nn.GELU(),
        M.DistributedConv2d(4, 2, 3, "cpu", (mesh["sh"], mesh["sw"]), mesh["col"], padding=1),
    )


def _worker_marks_and_sync(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    P = jb.parallel
    p = torch.nn.Parameter(torch.ones(3))
    P.mark_replicated(p, [mesh["sh"], None, mesh["col"]])       # None / size-1 dropped
    assert len(P.replica_groups(p)) == 1
    with pytest.raises(RuntimeError):
        P.mark_replicated(p, mesh["sw"])
    P.mark_replicated(p, [mesh["sw"], mesh["sh"]], extend=True)   # same rank set is skipped
    assert len(P.replica_groups(p)) == 2
    with pytest.raises(ValueError):
        P.mark_replicated(p, mesh["model"], extend=True)          # overlaps the marked groups
    # sync_grad sums over sh x sw
    (q,) = P.sync_grad(p)
    (q * (rank + 1.0)).sum().backward()
    assert_close(p.grad, torch.full((3,), 10.0), "sync_grad sum", 0, 0)
    with torch.no_grad():
        assert P.sync_grad(p)[0] is p
    assert P.sync_grad(None, torch.ones(2))[0] is None
    # broadcast_replicas / divergence / consistency checks
    lin = torch.nn.Linear(2, 2)
    for t in lin.parameters():
        P.mark_replicated(t, [mesh["sh"], mesh["sw"]])
    failed = False
    try:
        jb.debug.assert_replica_consistency(lin, mesh)
    except AssertionError:
        failed = True
    assert all_ok(failed), "different seeds must be detected on every rank"
    P.broadcast_replicas(lin)
    jb.debug.assert_replica_consistency(lin, mesh)
    out = P.synced_call(lin, torch.ones(1, 2) * (rank + 1))
    out.sum().backward()
    assert_close(lin.bias.grad, torch.full((2,), 4.0), "synced_call bias grad", 0, 0)
    # parameter counting: replicas once
    model = _tiny_model(mesh)
    serial = 2 * 4 * 9 + 4 + 4 * 2 * 9 + 2
    assert jb.debug.count_parameters(model, mesh) == serial
    assert jb.debug.count_parameters(model) == serial
    # clipping equals torch on the unsharded model
    for norm in (2.0, 1.0, 3.0, float("inf")):
        model.zero_grad()
        x = torch.randn(1, 2, 4, 4)
        model(x).square().sum().backward()
        ref = [p_.grad.clone() for p_ in model.parameters()]
        expect = torch.nn.utils.clip_grad_norm_([g.clone().requires_grad_() for g in ref], 1e9, norm)  # dummy call
        total = jb.parallel.clip_grad_norm_(model.parameters(), 0.5, mesh["model"], norm)
        vec = torch.cat([g.reshape(-1) for g in ref])
        want = vec.abs().max() if norm == float("inf") else vec.norm(norm)
        assert_close(total, want, f"clip total norm {norm}", 1e-5, 1e-6)
        coef = min(1.0, 0.5 / (float(want) + 1e-6))
        assert_close(next(model.parameters()).grad, ref[0] * coef, f"clip scale {norm}", 1e-5, 1e-7)


def _train(model, mesh, steps, data_seed, dp=None):
    import jigsaw_b200 as jb

    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    spec = {2: mesh["sh"], 3: mesh["sw"]}
    for step in range(steps):
        g = torch.Generator().manual_seed(data_seed(step))
        x = torch.randn(2, 2, 8, 8, generator=g)
        y = torch.randn(2, 2, 8, 8, generator=g)
        loss = loss_fn(model(split(x, spec)), split(y, spec))
        opt.zero_grad()
        loss.backward()
        opt.step()
    return loss.item()


def _worker_ddp(rank, world, joint):
    import jigsaw_b200 as jb
    import torch.distributed as dist

    mesh = jb.make_process_mesh({"dp": 2, "sh": 2, "sw": 1, "col": 1}, model_parallel_axes=("sh", "sw", "col"))
    model = _tiny_model(mesh)
    ddp = jb.parallel.wrap_ddp(model, mesh, joint_hook=joint)
    dp_rank = mesh["dp"].rank()
    _train(ddp, mesh, 3, lambda s: 100 + 2 * s + dp_rank)
    jb.debug.assert_replica_consistency(ddp, mesh)
    # serial oracle: same init, both samples-streams averaged
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Conv2d(2, 4, 3, padding=1), torch.nn.GELU(), torch.nn.Conv2d(4, 2, 3, padding=1))
    opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    for step in range(3):
        losses = []
        for d in range(2):
            g = torch.Generator().manual_seed(100 + 2 * step + d)
            x = torch.randn(2, 2, 8, 8, generator=g)
            y = torch.randn(2, 2, 8, 8, generator=g)
            losses.append(torch.nn.functional.mse_loss(ref(x), y))
        opt.zero_grad()
        (sum(losses) / 2).backward()
        opt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert_close(p.data, q.data, f"ddp(joint={joint}) parameters vs serial", 1e-4, 1e-5)
    if joint:
        state = getattr(ddp, "_jigsaw_joint_state")
        w = model[0].weight
        assert state.reduces(w) and state.group_of(w).size() == 4
        assert state.factor(jb.parallel.replica_groups(w)) == 2.0


def _worker_ddp_guards(rank, world):
    import jigsaw_b200 as jb
    from torch.nn.parallel import DistributedDataParallel as DDP

    mesh = jb.make_process_mesh({"dp": 2, "sh": 2, "sw": 1, "col": 1}, model_parallel_axes=("sh", "sw", "col"))
    model = _tiny_model(mesh)
    with pytest.raises(TypeError):
        jb.parallel.wrap_ddp(model, mesh, process_group=mesh["dp"])
    with pytest.raises(KeyError):
        jb.parallel.wrap_ddp(model, mesh, dp_key="nope")
    bad = DDP(model)                                  # default group spans the tiles: refused in the first forward
    with pytest.raises(RuntimeError, match="spans model-parallel"):
        bad(torch.randn(1, 2, 4, 4))
    model2 = _tiny_model(mesh, seed=1)
    with torch.no_grad():
        if mesh["sh"].rank() == 1:
            model2[0].weight.add_(1.0)                # diverged replica
    with pytest.raises(RuntimeError, match="differ across their replica groups"):
        jb.parallel.check_ddp(DDP(model2, process_group=mesh["dp"]))


def _worker_mutation(rank, world):
    """With gradient sync disabled the parity check must FAIL (the switch is read at import)."""
    os.environ["JIGSAW_DISABLE_GRAD_SYNC"] = "1"
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": 2, "sw": 1, "col": 1})
    model = _tiny_model(mesh)
    x = torch.randn(1, 2, 8, 8)
    model(split(x, {2: mesh["sh"]})).sum().backward()
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Conv2d(2, 4, 3, padding=1), torch.nn.GELU(), torch.nn.Conv2d(4, 2, 3, padding=1))
    ref(x).sum().backward()
    same = torch.allclose(model[0].weight.grad, ref[0].weight.grad, atol=1e-5)
    assert all_ok(not same), "gradients matched although the sync was disabled"


def test_marks_sync_clip_debug():
    run_distributed(_worker_marks_and_sync, 4)


def test_ddp_in_graph_mode_matches_serial():
    run_distributed(_worker_ddp, 4, False)


def test_ddp_joint_hook_matches_serial():
    run_distributed(_worker_ddp, 4, True)


def test_ddp_guards():
    run_distributed(_worker_ddp_guards, 4)


def test_disabling_grad_sync_is_detected():
    run_distributed(_worker_mutation, 2)


def _worker_accumulate(rank, world):
    """Gradient accumulation over three micro-batches: with ``no_grad_sync`` + one ``reduce_replica_grads``
    the gradients equal those of three synchronised backward passes, with a third of the all-reduces."""
    import torch.distributed as dist

    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    spec = {2: mesh["sh"], 3: mesh["sw"]}
    torch.manual_seed(5)
    batches = [(torch.randn(2, 2, 8, 8), torch.randn(2, 2, 8, 8)) for _ in range(3)]
    calls = {"n": 0}
    plain = dist.all_reduce

    def counting(*a, **k):
        calls["n"] += 1
        return plain(*a, **k)

    grads = []
    for deferred in (False, True):
        model = _tiny_model(mesh)
        dist.all_reduce = counting
        calls["n"] = 0
        try:
            if deferred:
                with jb.parallel.no_grad_sync():
                    for x, y in batches:
                        loss_fn(model(split(x, spec)), split(y, spec)).backward()
                jb.parallel.reduce_replica_grads(model)
            else:
                for x, y in batches:
                    loss_fn(model(split(x, spec)), split(y, spec)).backward()
        finally:
            dist.all_reduce = plain
        grads.append(([p.grad.clone() for p in model.parameters()], calls["n"]))
    (g_sync, n_sync), (g_acc, n_acc) = grads
    for a, b in zip(g_sync, g_acc):
        assert_close(b, a, "accumulated gradient", 1e-6, 1e-7)
    assert n_acc < n_sync, (n_acc, n_sync)


def test_gradient_accumulation_with_one_reduction():
    run_distributed(_worker_accumulate, 4)


def _worker_overlapped_sync(rank, world):
    """Bucketed reduction under the backward pass gives the gradients of the in-graph mode whatever the bucket
    size (up to the summation order of the transport, which depends on where an element sits in its bucket);
    gradient accumulation wraps only the last micro-batch."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    P = jb.parallel

    def build():
        model = _tiny_model(mesh)
        with torch.no_grad():
            for i, p in enumerate(model.parameters()):
                p.copy_(torch.randint(-2, 3, p.shape, generator=torch.Generator().manual_seed(100 + i)).float())
        return model

    def data(step):
        g = torch.Generator().manual_seed(10 * rank + step)
        return torch.randint(-2, 3, (1, 2, 4, 4), generator=g).float(), torch.randint(-2, 3, (1, 2, 4, 4), generator=g).float()

    ref = build()
    x, gy = data(0)
    ref(x).backward(gy)
    want = [p.grad.clone() for p in ref.parameters()]
    for bucket_bytes in (1, 64, 1 << 20):
        model = build()
        with P.OverlappedGradSync(model, bucket_bytes=bucket_bytes) as sync:
            model(x).backward(gy)
        assert sync.launched >= (4 if bucket_bytes == 1 else 1)
        for (n, p), w in zip(model.named_parameters(), want):
            assert all_ok(torch.allclose(p.grad, w, rtol=1e-5, atol=1e-5 * float(w.abs().max()))), f"bucket {bucket_bytes}: {n}"
    # accumulation over two micro-batches: the first under no_grad_sync, the second under the overlapped reduction
    ref = build()
    for step in range(2):
        x, gy = data(step)
        ref(x).backward(gy)
    want = [p.grad.clone() for p in ref.parameters()]
    model = build()
    x, gy = data(0)
    with P.no_grad_sync():
        model(x).backward(gy)
    x, gy = data(1)
    with P.OverlappedGradSync(model, bucket_bytes=128):
        model(x).backward(gy)
    for (n, p), w in zip(model.named_parameters(), want):
        assert all_ok(torch.allclose(p.grad, w, rtol=1e-5, atol=1e-5 * float(w.abs().max()))), f"accumulation: {n}: {float((p.grad - w).abs().max())} of {float(w.abs().max())}"
    # after the context the in-graph mode is back
    model = build()
    x, gy = data(0)
    model(x).backward(gy)
    ref = build()
    ref(x).backward(gy)
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.equal(p.grad, q.grad)
    with pytest.raises(RuntimeError):
        sync = P.OverlappedGradSync(model)
        with sync:
            with sync:
                pass


def test_overlapped_grad_sync_matches_the_in_graph_mode():
    run_distributed(_worker_overlapped_sync, 4)
