"""Attention layers under ``torch.vmap``: one layer over a stack of inputs, and an ensemble as stacked member
weights through ``functional_call``, against loops over the members.  Head-parallel, ring (layer input or K/V
circulating, chunks kept or fetched again), Ulysses.  Under ``vmap`` the ring folds the ensemble axis in front
of the batch axes, so one schedule of exchanges serves all members; with member weights K/V circulate, because
each member has projected its own.

Reference behaviours covered: tests/modules/attention/test_te_vmap_ensemble.py (forward and gradients of the
vmapped layer and of the stacked ensemble against loops; the ring case, which is refused there, runs here).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed

CASES = {
    "heads_only": ({"row": 1, "col": 4}, dict()),
    "heads_and_tokens": ({"row": 2, "col": 2}, dict()),
    "ring_x": ({"row": 4, "col": 1}, dict(ring=True, send_in_forward="x")),
    "ring_kv_local": ({"row": 4, "col": 1}, dict(ring=True, send_in_forward="kv", save_scope="local")),
    "ring_kv_heads": ({"row": 2, "col": 2}, dict(ring=True, send_in_forward="kv")),
    "ring_hybrid_gather": ({"row": 4, "col": 1}, dict(ring=True, send_in_forward="kv", send_op="hybrid", intra_size=2,
                                                      send_backward="gather_dkv")),
    "ulysses": ({"row": 2, "col": 2}, dict(ulysses=True)),
}
MEMBERS, DIM, HEADS, SEQ = 2, 8, 4, 8


def _layer(mesh, options, seed):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import RingAttentionConfig

    options = dict(options)
    ring, ulysses = options.pop("ring", False), options.pop("ulysses", False)
    config = RingAttentionConfig(device="cpu", attn_backend="math", **options) if ring else None
    jb.launch.set_all_seeds(seed * 11 + mesh["col"].rank())
    layer = jb.modules.DistributedAttention(DIM, 2 * DIM, DIM, HEADS, mesh["col"].rank(), "cpu", mesh["row"], mesh["col"],
                                            qk_norm=not ring or options.get("send_in_forward") == "kv", ring=ring,
                                            ulysses=ulysses, attn_backend="math", config=config)
    jb.parallel.broadcast_replicas(layer)
    return layer


def _worker(rank, world, case, member_weights):
    import jigsaw_b200 as jb
    from torch.func import functional_call, stack_module_state

    axes, options = CASES[case]
    mesh = jb.make_process_mesh(axes)
    x = torch.randn(MEMBERS, 3, SEQ // mesh["row"].size(), DIM // mesh["col"].size(),
                    generator=torch.Generator().manual_seed(40 + rank)).requires_grad_(True)
    if member_weights:
        members = [_layer(mesh, options, s) for s in range(MEMBERS)]
        base = _layer(mesh, options, 77)
        params, buffers = stack_module_state(members)
        params = {k: v.detach().clone().requires_grad_(True) for k, v in params.items()}
        got = torch.vmap(lambda p, b, xi: functional_call(base, (p, b), (xi,)))(params, buffers, x)
        want = torch.stack([m(xi) for m, xi in zip(members, x)])
    else:
        base = _layer(mesh, options, 3)
        got = torch.vmap(base)(x)
        want = torch.stack([base(xi) for xi in x])
    tag = f"{case}, {'member weights' if member_weights else 'one layer'}"
    assert_close(got, want, f"{tag}: output", 1e-4, 1e-5)
    weights = torch.randn(want.shape, generator=torch.Generator().manual_seed(8 + rank))
    named = dict(base.named_parameters())
    if member_weights:
        (got * weights).sum().backward()
        gx, x.grad = x.grad.clone(), None
        (want * weights).sum().backward()
        assert_close(gx, x.grad, f"{tag}: input gradient", 1e-3, 1e-5)
        for n, p in params.items():                     # functional_call hands over tensors without replica marks
            jb.parallel.mark_replicated(p, jb.parallel.replica_groups(named[n]))
        jb.parallel.reduce_replica_grads(params.values())
        for n, p in params.items():
            want_grad = torch.stack([dict(m.named_parameters())[n].grad for m in members])
            assert_close(p.grad, want_grad, f"{tag}: gradient of {n}", 1e-3, 1e-5)
    else:
        leaves = [x, *named.values()]
        grads = torch.autograd.grad((got * weights).sum(), leaves)
        wants = torch.autograd.grad((want * weights).sum(), leaves)
        for g, w, n in zip(grads, wants, ["input", *named]):
            assert_close(g, w, f"{tag}: gradient of {n}", 1e-3, 1e-5)


@pytest.mark.parametrize("member_weights", [False, True], ids=["one_layer", "member_weights"])
@pytest.mark.parametrize("case", list(CASES))
def test_vmapped_attention_matches_the_loop(case, member_weights):
    run_distributed(_worker, 4, case, member_weights, timeout=300)
