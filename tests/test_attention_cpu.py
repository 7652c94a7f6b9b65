"""Attention parity on CPU/gloo ranks: ring (every topology / save scope / dK-dV routing),
Ulysses (flat and hierarchical), circulated-input mode, head-parallel projections, masks,
and conversion to / from the serial layer."""

import itertools

import pytest
import torch

from dist_utils import assert_close, run_distributed, split


def _serial_and_grads(att, x, mask=None):
    xr = x.clone().requires_grad_(True)
    y = att(xr, mask) if mask is not None else att(xr)
    gy = torch.randn(y.shape, generator=torch.Generator().manual_seed(7), dtype=y.dtype)
    y.backward(gy)
    return xr, y.detach(), gy


def _compare(layer, att, x, xr, y_ref, gy, mesh, what, tol=1e-9):
    row, col = mesh["row"], mesh["col"]
    spec = {1: row, 2: col}
    xl = split(x, spec).requires_grad_(True)
    y = layer(xl)
    assert_close(y, split(y_ref, spec), f"{what}: output", tol, tol)
    y.backward(split(gy, spec))
    assert_close(xl.grad, split(xr.grad, spec), f"{what}: dx", tol, tol)
    back = layer.convert_to_torch(mesh)
    assert_close(back.qkv.weight.data, att.qkv.weight.data, f"{what}: qkv round trip", 0, 0)
    # parameter gradients: compare through the merged layout
    C = col.size()
    gq = layer.qkv.weight.grad
    if C > 1:
        from jigsaw_b200._core.placement import gather_dim

        gq = gather_dim(gq, col, 1)
    heads_local = att.heads // C
    gq = gq.view(C, 3, heads_local, att.head_dim, att.in_dim).transpose(0, 1).reshape(3 * att.embed_dim, att.in_dim)
    assert_close(gq, att.qkv.weight.grad, f"{what}: dW_qkv", tol, tol)


def _worker_ring_policies(rank, world, send_op):
    """One schedule of visits with every way of keeping chunks, returning dK/dV and overlapping the exchange."""
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention, RingAttentionConfig

    mesh = jb.make_process_mesh({"row": 4, "col": 1})
    torch.manual_seed(0)
    att = Attention(8, 16, 8, 4, "cpu", dtype=torch.float64, attn_backend="math")
    x = torch.randn(2, 16, 8, dtype=torch.float64)
    for scope, back, overlap in itertools.product(("local", "global"), ("send_dkv", "gather_dkv"), (False, True)):
        cfg = RingAttentionConfig(device="cpu", send_in_forward="kv", send_op=send_op, save_scope=scope,
                                  send_backward=back, intra_size=2, attn_backend="math", overlap_comm=overlap)
        layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=True, config=cfg, attn_backend="math")
        att.zero_grad()
        xr, y_ref, gy = _serial_and_grads(att, x)
        _compare(layer, att, x, xr, y_ref, gy, mesh, f"ring {send_op}/{scope}/{back}/overlap={overlap}")


def _worker_ring(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention, RingAttentionConfig

    mesh = jb.make_process_mesh({"row": 4, "col": 1})
    torch.manual_seed(0)
    att = Attention(8, 16, 8, 4, "cpu", dtype=torch.float64, attn_backend="math")
    x = torch.randn(2, 16, 8, dtype=torch.float64)
    # the layer input circulates and K/V are re-projected on arrival
    cfg = RingAttentionConfig(device="cpu", send_in_forward="x", attn_backend="math")
    layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=True, config=cfg, attn_backend="math")
    att.zero_grad()
    xr, y_ref, gy = _serial_and_grads(att, x)
    _compare(layer, att, x, xr, y_ref, gy, mesh, "ring send_in_forward=X")
    # no-grad forward keeps nothing
    from jigsaw_b200.modules.attention import _ring

    kept = []
    plain_setup = _ring._RingAttention.setup_context
    _ring._RingAttention.setup_context = staticmethod(lambda ctx, inputs, output: (kept.append(dict(inputs[-1])), plain_setup(ctx, inputs, output))[1])
    try:
        layer(split(x, {1: mesh["row"]}).requires_grad_(True))
        assert len(kept) == 1 and kept[0]["saved_chunks"] is not None and len(kept[0]["saved_chunks"]) == mesh["row"].size()
        for mode in (torch.no_grad, torch.inference_mode):
            with mode():
                y = layer(split(x, {1: mesh["row"]}))
            assert_close(y, split(y_ref, {1: mesh["row"]}), f"ring under {mode.__name__}", 1e-9, 1e-9)
        assert kept[1:] == [{}, {}], "a forward pass without grad mode kept chunks for a backward pass that cannot come"
    finally:
        _ring._RingAttention.setup_context = plain_setup
    # guards
    with pytest.raises(ValueError):
        jb.modules.DistributedAttention(8, 16, 8, 4, 0, "cpu", mesh["col"], mesh["col"], ring=True)
    with pytest.raises(ValueError):
        jb.modules.DistributedAttention(8, 16, 8, 4, 0, "cpu", mesh["row"], mesh["col"], ring=True, ulysses=True)
    with pytest.raises(ValueError):
        RingAttentionConfig(device="cpu", send_op="nonsense")


def _worker_ulysses(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention

    mesh = jb.make_process_mesh({"row": 4, "col": 1})
    torch.manual_seed(1)
    att = Attention(8, 32, 8, 8, "cpu", dtype=torch.float64, attn_backend="math", qk_norm=True)
    x = torch.randn(2, 16, 8, dtype=torch.float64)
    xr, y_ref, gy = _serial_and_grads(att, x)
    layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=False, ulysses=True, attn_backend="math")
    _compare(layer, att, x, xr, y_ref, gy, mesh, "ulysses")
    for scope in ("local", "global"):
        att.zero_grad()
        xr, y_ref, gy = _serial_and_grads(att, x)
        layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=False, ulysses=True, ulysses_intra_size=2,
                                            ulysses_inter_save_scope=scope, attn_backend="math")
        _compare(layer, att, x, xr, y_ref, gy, mesh, f"hierarchical ulysses {scope}")
    with pytest.raises(ValueError):
        jb.modules.DistributedAttention(8, 24, 8, 6, 0, "cpu", mesh["row"], mesh["col"], ulysses=True)


def _worker_heads(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    torch.manual_seed(2)
    att = Attention(8, 16, 12, 4, "cpu", dtype=torch.float64, attn_backend="math")
    x = torch.randn(2, 8, 8, dtype=torch.float64)
    xr, y_ref, gy = _serial_and_grads(att, x)
    layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=True, attn_backend="math")
    assert layer.heads == 2 and isinstance(layer.qkv, jb.modules.DistributedLinear)
    _compare(layer, att, x, xr, y_ref, gy, mesh, "ring + head parallel")
    att.zero_grad()
    xr, y_ref, gy = _serial_and_grads(att, x)
    layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=False, ulysses=True, attn_backend="math")
    _compare(layer, att, x, xr, y_ref, gy, mesh, "ulysses + head parallel")
    # window attention: no sequence parallelism, extra window axis, additive mask
    mesh1 = {"row": mesh["col"], "col": mesh["col"]}
    xw = torch.randn(2, 3, 8, 8, dtype=torch.float64)
    mask = torch.randn(3, 1, 8, 8, dtype=torch.float64)
    att.zero_grad()
    xr = xw.clone().requires_grad_(True)
    y_ref = att(xr, mask)
    layer = jb.modules.DistributedAttention(8, 16, 12, 4, 0, "cpu", mesh["row"], mesh["col"], attn_backend="math",
                                            dtype=torch.float64)
    conv = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=False, attn_backend="math")
    y = conv(split(xw, {3: mesh["col"]}), mask)
    assert_close(y, split(y_ref.detach(), {3: mesh["col"]}), "window attention with mask", 1e-9, 1e-9)
    assert "ring=False" in repr(conv) and conv.get_parameter_count() == 0


@pytest.mark.parametrize("send_op", ["ring", "broadcast", "hybrid", "hybrid_broadcast"])
def test_ring_attention_policies(send_op):
    run_distributed(_worker_ring_policies, 4, send_op, timeout=400)


def test_ring_with_circulating_input_without_grad_and_guards():
    run_distributed(_worker_ring, 4, timeout=400)


def test_ulysses_and_hierarchical():
    run_distributed(_worker_ulysses, 4)


def test_head_parallel_and_window_attention():
    run_distributed(_worker_heads, 4)


@pytest.mark.parametrize("parts", [2, 4])
def test_fused_ulysses_projection_layouts(parts):
    """Layout algebra of the projection with the exchange in its epilogue, with the ranks emulated by a
    loop: column part ``p`` of ``x_r @ head_group_major(w).T`` is what rank ``r`` stores into rank ``p``'s
    inbox; the inbox must read as the head shard of the gathered q, k, v, and the helpers of the
    backward pass must reproduce autograd's gradients of the unfused formulation."""
    from jigsaw_b200.ops.ulysses_fused import from_head_group_major, grad_columns, head_group_major, inbox_to_qkv

    torch.manual_seed(0)
    b, sl, heads, d, K = 2, 3, 8, 4, 5
    hl, cols = heads // parts, 3 * (heads // parts) * d
    w = torch.randn(3 * heads * d, K, dtype=torch.float64, requires_grad=True)
    xs = [torch.randn(b, sl, K, dtype=torch.float64, requires_grad=True) for _ in range(parts)]
    # unfused formulation: project, split heads, gather the sequence, keep this rank's heads
    full = torch.cat([(x @ w.T).view(b, sl, 3, heads, d).permute(2, 0, 1, 3, 4) for x in xs], dim=2)
    wp = head_group_major(w.detach(), parts, heads, d)
    assert torch.equal(from_head_group_major(wp, parts, heads, d), w.detach())
    slabs = [(x.detach().reshape(b * sl, K) @ wp.T) for x in xs]              # what each source rank's GEMM produces
    gs = []
    for p in range(parts):
        inbox = torch.stack([s[:, p * cols:(p + 1) * cols] for s in slabs]).contiguous()
        out = inbox_to_qkv(inbox, parts, b, sl, hl, d)
        ref = full[..., p * hl:(p + 1) * hl, :]
        assert torch.allclose(out, ref.detach(), atol=1e-12), f"forward layout of rank {p}"
        gs.append(torch.randn_like(out))
    g_full = torch.cat(gs, dim=3)                                             # (3, b, s, heads, d)
    grads = torch.autograd.grad(full, [w, *xs], g_full)
    dw = torch.zeros_like(wp)
    for r, x in enumerate(xs):
        back = g_full[:, :, r * sl:(r + 1) * sl].contiguous()                 # what the inverse exchange returns to rank r
        g2 = grad_columns(back, parts, b, sl, hl, d)
        assert torch.allclose((g2 @ wp).view(b, sl, K), grads[1 + r], atol=1e-12), f"input gradient of rank {r}"
        dw += g2.T @ x.detach().reshape(b * sl, K)
    assert torch.allclose(from_head_group_major(dw, parts, heads, d), grads[0], atol=1e-12), "weight gradient"


@pytest.mark.parametrize("parts", [2, 4])
def test_fused_ulysses_output_projection_layouts(parts):
    """Layout algebra of the output projection whose operand loads do the head -> sequence exchange,
    ranks emulated by a loop: k-block part ``p`` of rank ``r``'s A operand is entry ``r`` of rank ``p``'s
    staging block; in the backward pass column part ``p`` of ``gy_r @ W`` is slab ``r`` of rank ``p``'s inbox."""
    from jigsaw_b200.ops.ulysses_fused import stage_for_owners

    torch.manual_seed(0)
    b, sl, hl, d, N = 2, 3, 2, 4, 6
    s, kp = parts * sl, hl * d
    w = torch.randn(N, parts * kp, dtype=torch.float64)
    os_ = [torch.randn(b, hl, s, d, dtype=torch.float64).transpose(1, 2).requires_grad_(True) for _ in range(parts)]   # (b, s, hl, d) views
    ys = []
    for r in range(parts):                                                    # unfused formulation on rank r
        mine = torch.cat([o[:, r * sl:(r + 1) * sl] for o in os_], dim=2)     # heads_to_seq: (b, sl, h, d)
        ys.append(mine.reshape(b * sl, parts * kp) @ w.T)
    staged = [stage_for_owners(o.detach(), parts).contiguous() for o in os_]
    for r in range(parts):
        a = torch.cat([staged[p][r].reshape(b * sl, kp) for p in range(parts)], dim=1)
        assert torch.allclose(a @ w.T, ys[r].detach(), atol=1e-12), f"forward operand of rank {r}"
    gys = [torch.randn_like(y) for y in ys]
    grads = torch.autograd.grad(ys, os_, gys)
    full = [g @ w for g in gys]                                               # (M, P * kp) on every source rank
    for p in range(parts):
        inbox = torch.stack([f[:, p * kp:(p + 1) * kp] for f in full]).contiguous()
        do = inbox.view(parts, b, sl, hl, d).permute(1, 0, 2, 3, 4).reshape(b, s, hl, d)
        assert torch.allclose(do, grads[p], atol=1e-12), f"gradient of rank {p}'s heads"


def _worker_ring_dropout(rank, world):
    """Ring attention with dropout: the masks are reproducible from the seed (forward and the chunk
    re-visits of the backward pass use the same ones), so for a fixed seed the layer is linear in the values
    and its gradient matches a finite difference taken under the same seed."""
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention, RingAttentionConfig

    mesh = jb.make_process_mesh({"row": 4, "col": 1})
    torch.manual_seed(0)
    att = Attention(8, 16, 8, 4, "cpu", dropout_p=0.3, dtype=torch.float64, attn_backend="math")
    x = torch.randn(2, 16, 8, dtype=torch.float64)
    xl = split(x, {1: mesh["row"]})
    for scope in ("local", "global"):
        cfg = RingAttentionConfig(device="cpu", send_in_forward="kv", save_scope=scope, attn_backend="math")
        layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=True, config=cfg, attn_backend="math")
        layer.train()

        def run(inp):
            torch.manual_seed(123)                       # the layer draws its base seed from the global generator
            return layer(inp)

        y1, y2 = run(xl), run(xl)
        assert_close(y2.detach(), y1.detach(), f"{scope}: same seed, same masks", 0, 0)
        layer.eval()
        assert float((layer(xl) - y1).abs().max()) > 1e-3, "dropout changed nothing"
        layer.train()
        # directional derivative with respect to the input against autograd, under the same seed
        xg = xl.clone().requires_grad_(True)
        g = torch.randn_like(y1)
        (run(xg) * g).sum().backward()
        d = torch.randn_like(xl)
        eps = 1e-6
        fd = ((run(xl + eps * d) - run(xl - eps * d)) * g).sum() / (2 * eps)
        # the input of one rank feeds the outputs of all ranks (it is their K / V): sum both sides over the ring
        import torch.distributed as dist

        lhs = fd.detach().reshape(1)
        rhs = (xg.grad * d).sum().reshape(1)
        dist.all_reduce(lhs, group=mesh["row"])
        dist.all_reduce(rhs, group=mesh["row"])
        assert_close(rhs, lhs, f"{scope}: gradient under dropout", 1e-5, 1e-7)


def test_ring_attention_dropout_is_reproducible_and_differentiable():
    run_distributed(_worker_ring_dropout, 4)


def _worker_attention_reshard(rank, world):
    """``DistributedAttention.reshard_parameters`` over three meshes: on every mesh the layer (heads per rank,
    groups, ring / Ulysses or dense attention where the sequence is not split) reproduces the serial layer."""
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention, RingAttentionConfig

    meshes = [jb.make_process_mesh({"row": 2, "col": 2}), jb.make_process_mesh({"row": 1, "col": 4}),
              jb.make_process_mesh({"row": 4, "col": 1}), jb.make_process_mesh({"row": 2, "col": 2})]
    torch.manual_seed(0)
    att = Attention(8, 16, 8, 4, "cpu", dtype=torch.float64, attn_backend="math")
    x = torch.randn(2, 16, 8, dtype=torch.float64)
    y_ref = att(x).detach()
    for mode in ("ring", "ulysses"):
        cfg = RingAttentionConfig(device="cpu", send_in_forward="kv", attn_backend="math") if mode == "ring" else None
        layer = Attention.convert_to_jigsaw(att, meshes[0], "cpu", ring=mode == "ring", ulysses=mode == "ulysses",
                                            attn_backend="math", config=cfg)
        for a, b in zip(meshes[:-1], meshes[1:]):
            layer.reshard_parameters(a, b)
            cuts = {1: b["row"], 2: b["col"]}
            y = layer(split(x, cuts))
            assert_close(y.detach(), split(y_ref, cuts), f"{mode}: output on a {b['row'].size()}x{b['col'].size()} mesh", 1e-9, 1e-9)
            split_seq = b["row"].size() > 1
            assert (layer.ring, layer.ulysses) == (mode == "ring" and split_seq, mode == "ulysses" and split_seq)
        # a mesh that does not divide the heads is refused and changes nothing
        odd = jb.make_process_mesh({"row": 1, "col": 4})
        small = Attention.convert_to_jigsaw(Attention(8, 12, 8, 2, "cpu", dtype=torch.float64, attn_backend="math"), meshes[0], "cpu",
                                            ring=False, attn_backend="math")
        xs = split(x, {1: meshes[0]["row"], 2: meshes[0]["col"]})
        before = small(xs).detach()
        with pytest.raises(ValueError):
            small.reshard_parameters(meshes[0], odd)
        assert_close(small(xs).detach(), before, "after a refused reshard", 0, 0)


def test_attention_reshard_over_meshes():
    run_distributed(_worker_attention_reshard, 4)


def _worker_ulysses_exchange(rank, world):
    """The two exchanges of Ulysses on their own: sequence pieces become head pieces and back."""
    import torch.distributed as dist
    from jigsaw_b200.modules.attention._ulysses import heads_to_seq, seq_to_heads

    group = dist.group.WORLD
    b, s_local, heads, d = 2, 3, 2 * world, 5
    x = torch.randn(b, s_local, heads, d, generator=torch.Generator().manual_seed(rank), dtype=torch.float64)
    whole_seq = seq_to_heads(x, group)                                   # (b, s, heads / P, d)
    assert tuple(whole_seq.shape) == (b, s_local * world, heads // world, d)
    everyone = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(everyone, x)
    mine = slice(rank * (heads // world), (rank + 1) * (heads // world))
    want = torch.cat([piece[:, :, mine] for piece in everyone], dim=1)  # sequence in rank order, my window of heads
    assert_close(whole_seq, want, "sequence gathered, heads scattered", 0, 0)
    assert_close(heads_to_seq(whole_seq, group), x, "there and back", 0, 0)
    stacked = torch.stack((x, 2 * x, 3 * x))                             # q, k, v in one exchange
    got = seq_to_heads(stacked, group)
    assert_close(got, torch.stack((want, 2 * want, 3 * want)), "stacked q, k, v", 0, 0)
    leaf = x.clone().requires_grad_(True)
    seed = torch.randn(whole_seq.shape, generator=torch.Generator().manual_seed(50 + rank), dtype=torch.float64)
    (grad,) = torch.autograd.grad(seq_to_heads(leaf, group), leaf, seed)
    assert_close(grad, heads_to_seq(seed, group), "the backward of one exchange is the other", 0, 0)


def test_ulysses_exchanges_round_trip():
    run_distributed(_worker_ulysses_exchange, 4)
