"""Attention dropout: the math core against a hand-written masked softmax (forward and backward replay the same mask
from the seed), seed derivation per (rank, chunk), eval mode, and the distributed layers (ring and Ulysses replay their
masks between forward and backward; ranks draw independent masks under one shared seed).

Reference behaviours covered: tests/modules/attention/test_dropout.py:56-134 (math core), :136-147 (seed
derivation), :149-248 (eval / train mode, serial and distributed), :639-818 (replay and independence in the
distributed layers).
"""

import torch

from dist_utils import all_ok, assert_close, run_distributed, split


def test_math_core_replays_its_mask():
    from jigsaw_b200.modules.attention._cores import MathCore, _dropout_mask

    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 3, 5, 4, generator=g, dtype=torch.float64) for _ in range(3))
    scale, p, seed = 0.5, 0.25, 1234
    out, lse, state = MathCore.forward(q, k, v, scale, p, seed)
    probs = torch.softmax(q @ k.transpose(-1, -2) * scale, -1)
    mask = _dropout_mask(probs.shape, p, seed, probs.device).double()
    assert torch.allclose(out, (probs * mask) @ v, atol=1e-12)
    assert torch.allclose(lse, torch.logsumexp(q @ k.transpose(-1, -2) * scale, -1), atol=1e-12)
    keep = (mask > 0).double().mean()
    assert abs(float(keep) - (1 - p)) < 0.15 and torch.all((mask == 0) | torch.isclose(mask, torch.tensor(1 / (1 - p), dtype=torch.float64)))
    # backward with the saved state equals autograd through the same masked softmax
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = (torch.softmax(qa @ ka.transpose(-1, -2) * scale, -1) * mask) @ va
    dout = torch.randn(out.shape, generator=g, dtype=torch.float64)
    ref.backward(dout)
    dq, dk, dv = MathCore.backward(dout, q, k, v, out, lse, scale, p, state)
    for got, want, name in ((dq, qa.grad, "dq"), (dk, ka.grad, "dk"), (dv, va.grad, "dv")):
        assert torch.allclose(got, want, atol=1e-10), name
    # another seed is another mask; without dropout the seed does not matter
    other, _, _ = MathCore.forward(q, k, v, scale, p, seed + 1)
    assert not torch.allclose(other, out)
    a, _, _ = MathCore.forward(q, k, v, scale, 0.0, 1)
    b, _, _ = MathCore.forward(q, k, v, scale, 0.0, 2)
    assert torch.equal(a, b)


def test_chunk_seeds_are_deterministic_and_distinct():
    from jigsaw_b200.modules.attention._cores import chunk_seed

    assert chunk_seed(42, 1, 2) == chunk_seed(42, 1, 2)
    seeds = {chunk_seed(base, rank, chunk) for base in (1, 2) for rank in range(4) for chunk in range(4)}
    assert len(seeds) == 32, "every (base, rank, chunk) must get its own seed"
    assert all(0 <= s < 2**31 - 1 for s in seeds)


def test_eval_mode_disables_dropout_in_the_serial_layer():
    from jigsaw_b200.modules.attention import Attention

    torch.manual_seed(0)
    att = Attention(8, 16, 8, 4, "cpu", dropout_p=0.5, dtype=torch.float64, attn_backend="math")
    clean = Attention(8, 16, 8, 4, "cpu", dropout_p=0.0, dtype=torch.float64, attn_backend="math")
    clean.load_state_dict(att.state_dict())
    x = torch.randn(2, 6, 8, dtype=torch.float64)
    att.eval()
    assert torch.equal(att(x), clean(x))
    att.train()
    a, b = att(x), att(x)
    assert not torch.allclose(a, b), "two training passes drew the same mask"


def _worker_distributed_dropout(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist
    from jigsaw_b200.modules.attention import Attention, RingAttentionConfig

    mesh = jb.make_process_mesh({"row": 4, "col": 1})
    row = mesh["row"]
    torch.manual_seed(0)
    att = Attention(8, 32, 8, 8, "cpu", dropout_p=0.4, dtype=torch.float64, attn_backend="math")
    clean = Attention(8, 32, 8, 8, "cpu", dropout_p=0.0, dtype=torch.float64, attn_backend="math")
    clean.load_state_dict(att.state_dict())
    x = torch.randn(2, 16, 8, dtype=torch.float64)
    xl = split(x, {1: row})
    cfg = RingAttentionConfig(device="cpu", send_in_forward="kv", attn_backend="math")
    for mode, kw in (("ring", dict(ring=True, config=cfg)), ("ulysses", dict(ring=False, ulysses=True))):
        layer = Attention.convert_to_jigsaw(att, mesh, "cpu", attn_backend="math", **kw)
        ref = Attention.convert_to_jigsaw(clean, mesh, "cpu", attn_backend="math", **kw)
        layer.eval()
        assert_close(layer(xl), ref(xl).detach(), f"{mode}: eval mode equals zero dropout", 0, 0)
        layer.train()

        def run(inp, seed=7):
            torch.manual_seed(seed)                              # the same shared seed on every rank
            return layer(inp)

        y = run(xl)
        assert_close(run(xl).detach(), y.detach(), f"{mode}: the seed fixes the masks", 0, 0)
        assert all_ok(not torch.allclose(run(xl, seed=8), y)), f"{mode}: another seed must give other masks"
        # replay: for a fixed seed the layer is linear in v, hence in x through v only up to softmax terms; the
        # gradient must match a finite difference taken under the same seed, which fails if backward drew new masks
        xg = xl.clone().requires_grad_(True)
        g = torch.randn(y.shape, generator=torch.Generator().manual_seed(rank), dtype=torch.float64)
        (run(xg) * g).sum().backward()
        d = torch.randn(xl.shape, generator=torch.Generator().manual_seed(100 + rank), dtype=torch.float64)
        eps = 1e-6
        fd = (((run(xl + eps * d) - run(xl - eps * d)) * g).sum() / (2 * eps)).detach().reshape(1)
        an = (xg.grad * d).sum().reshape(1)
        dist.all_reduce(fd, group=row)
        dist.all_reduce(an, group=row)
        assert_close(an, fd, f"{mode}: backward replays the forward masks", 1e-5, 1e-7)
        # independence: identical inputs on every rank and one shared seed must still give different outputs per
        # rank (each rank mixes its rank and the chunk into the seed), otherwise the masks would be correlated
        same = torch.randn(2, 4, 8, generator=torch.Generator().manual_seed(3), dtype=torch.float64)
        out = run(same)
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out.detach().contiguous(), group=row)
        layer.eval()
        plain = layer(same)
        layer.train()
        dev = [float((o - plain).abs().max()) for o in gathered]     # what dropout changed, per rank
        assert all(v > 1e-6 for v in dev), f"{mode}: dropout changed nothing on some rank"
        distinct = len({round(v, 9) for v in dev})
        assert all_ok(distinct >= world - 1), f"{mode}: ranks drew the same masks under one seed ({dev})"


def test_distributed_layers_replay_and_decorrelate_their_masks():
    run_distributed(_worker_distributed_dropout, 4, timeout=300)
