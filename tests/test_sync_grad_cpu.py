"""``mark_replicated``, ``sync_grad``, ``synced_parameters`` and ``synced_call`` in isolation: which groups a mark
keeps, what the in-graph sum adds up, how many collectives it issues, repeated use, unused outputs, ``vmap``,
micro-batches, foreign modules.

Reference behaviours covered: tests/test_parallel.py:52-108 (marks), :111-201 (sync_grad), :203-213 (accumulation),
:215-256 (synced parameters and calls).
"""

import pytest
import torch

from dist_utils import run_distributed

BASE = torch.tensor([1.0, 2.0, 3.0])


def _worker_sync(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist

    P = jb.parallel
    mesh = jb.make_process_mesh({"a": 2, "b": 2}, model_parallel_axes=("a", "b"))
    W = dist.group.WORLD
    world_sum = float(sum(r + 1 for r in range(world)))
    scale = float(rank + 1)

    def param(dtype=torch.float32):
        return torch.nn.Parameter(torch.zeros(3, dtype=dtype))

    def loss(q):
        return (q * BASE.to(q.dtype) * scale).sum()            # d loss / d q = BASE * (rank + 1)

    # ---- marks
    p = param()
    P.mark_replicated(p, mesh["a"])
    with pytest.raises(RuntimeError):
        P.mark_replicated(p, mesh["b"])                          # a second mark needs extend=True
    P.mark_replicated(p, mesh["b"], extend=True)
    assert P.replica_groups(p) == (mesh["a"], mesh["b"])
    P.mark_replicated(p, [mesh["b"], mesh["a"]], extend=True)    # groups over the same ranks are dropped
    assert len(P.replica_groups(p)) == 2
    with pytest.raises(ValueError):
        P.mark_replicated(p, W, extend=True)                     # overlaps what is marked already
    q = param()
    P.mark_replicated(q, mesh["a"], extend=True)                 # extend also marks an unmarked parameter
    assert P.replica_groups(q) == (mesh["a"],)
    r = param()
    P.mark_replicated(r, [None, mesh["b"]])
    assert P.replica_groups(r) == (mesh["b"],) and P.replica_groups(param()) == () and P.replica_groups(None) == ()
    # ---- sums
    for groups, want in ((W, world_sum), ([mesh["a"], mesh["b"]], world_sum),
                         (mesh["b"], float(sum(m + 1 for m in dist.get_process_group_ranks(mesh["b"]))))):
        p = param()
        P.mark_replicated(p, groups)
        (s,) = P.sync_grad(p)
        loss(s).backward()
        assert torch.equal(p.grad, BASE * want), (groups, p.grad)
    # ---- pass-through cases issue no collective
    calls = []
    original = dist.all_reduce

    def counting(tensor, *a, **k):
        calls.append(tensor.dtype)
        return original(tensor, *a, **k)

    dist.all_reduce = counting
    try:
        marked, plain = param(), param()
        P.mark_replicated(marked, W)
        frozen = param().requires_grad_(False)
        P.mark_replicated(frozen, W)
        out = P.sync_grad(plain, None, frozen)
        assert out[0] is plain and out[1] is None and out[2] is frozen
        with torch.no_grad():
            assert P.sync_grad(marked)[0] is marked
        assert calls == []
        # one flattened collective per (groups, dtype) bucket
        a, b, c = param(), param(), param(torch.float64)
        for t in (a, b, c):
            P.mark_replicated(t, W)
        qa, qb, qc = P.sync_grad(a, b, c)
        (loss(qa) + loss(qb) + loss(qc)).backward()
        assert len(calls) == 2 and sorted(map(str, calls)) == ["torch.float32", "torch.float64"], calls
        for t in (a, b, c):
            assert torch.equal(t.grad.float(), BASE * world_sum)
    finally:
        dist.all_reduce = original
    # ---- a parameter routed twice: S(g1) + S(g2) = S(g1 + g2)
    p = param()
    P.mark_replicated(p, W)
    (q1,), (q2,) = P.sync_grad(p), P.sync_grad(p)
    (loss(q1) + 2 * loss(q2)).backward()
    assert torch.equal(p.grad, 3 * BASE * world_sum)
    # ---- an output that is not used gets a zero gradient (the flat buffer keeps its size on every rank)
    a, b = param(), param()
    for t in (a, b):
        P.mark_replicated(t, W)
    qa, _ = P.sync_grad(a, b)
    loss(qa).backward()
    assert torch.equal(a.grad, BASE * world_sum) and torch.equal(b.grad, torch.zeros(3))
    # ---- vmap over the input
    p = param()
    P.mark_replicated(p, W)

    def f(xi):
        (s,) = P.sync_grad(p)
        return loss(s * xi)

    torch.vmap(f)(torch.ones(4, 3)).sum().backward()
    assert torch.equal(p.grad, 4 * BASE * world_sum)
    # ---- every micro-batch is reduced on its own, never the running sum in .grad
    for micro in (1, 2, 3):
        p = param()
        P.mark_replicated(p, W)
        for _ in range(micro):
            (s,) = P.sync_grad(p)
            loss(s).backward()
        assert torch.equal(p.grad, micro * BASE * world_sum)
    # ---- foreign modules
    lin = torch.nn.Linear(3, 3)
    P.mark_replicated(lin.weight, W)
    synced = P.synced_parameters(lin)
    assert set(synced) == {"weight"} and synced["weight"] is not lin.weight
    lin = torch.nn.Linear(3, 1, bias=False)
    P.mark_replicated(lin.weight, W)
    x = BASE[None] * scale
    torch.func.functional_call(lin, P.synced_parameters(lin), (x,)).sum().backward()
    assert torch.equal(lin.weight.grad, BASE[None] * world_sum)
    lin = torch.nn.Linear(3, 1)
    lin.bias.data.zero_()
    P.mark_replicated(lin.weight, W)
    P.synced_call(lin, x).sum().backward()
    assert torch.equal(lin.weight.grad, BASE[None] * world_sum) and torch.equal(lin.bias.grad, torch.ones(1))
    attn = torch.nn.MultiheadAttention(3, 1, bias=False)
    P.mark_replicated(attn.in_proj_weight, W)
    xa = BASE[None, None]
    out, weights = P.synced_call(attn, xa, xa, xa, need_weights=False)
    assert out.shape == (1, 1, 3) and weights is None


def test_marks_and_in_graph_sums():
    run_distributed(_worker_sync, 4, timeout=300)
