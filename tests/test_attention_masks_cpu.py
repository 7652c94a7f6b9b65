"""``attn_mask`` in ``Attention`` and ``DistributedAttention``.

Shifted-window attention needs an arbitrary mask per window (tokens stitched together by the cyclic shift
must not see each other), broadcastable to ``(..., heads, seq, seq)``; a valid-length cut-off is not enough.
The dense core (``attn_backend`` ``sdpa`` / ``math``, no sequence parallelism) supports boolean and additive
masks; ring and Ulysses refuse a mask instead of ignoring it.

Reference behaviours covered: tests/modules/attention/test_attn_mask.py:131-212 (block mask = separate
attention, additive = boolean, blindness, gradients), :214-283 and :342-402 (arbitrary masks against an explicit
softmax, both backends, serial and head-parallel), :404-482 (ring / Ulysses reject a mask).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split

DIM, HEADS = 32, 4


def _block_mask(n0, n1):
    """Boolean block-diagonal mask: ``n0`` tokens of one region, ``n1`` of another, no sight across."""
    m = torch.zeros(n0 + n1, n0 + n1, dtype=torch.bool)
    m[:n0, :n0] = True
    m[n0:, n0:] = True
    return m


def _layer(backend="math", qk_norm=False, seed=0):
    from jigsaw_b200.modules.attention import Attention

    torch.manual_seed(seed)
    return Attention(DIM, DIM, DIM, HEADS, "cpu", dtype=torch.float64, attn_backend=backend, qk_norm=qk_norm)


def _explicit(att, x, mask):
    """Attention written out with an explicit softmax (the oracle of the arbitrary-mask cases)."""
    b, s, _ = x.shape
    qkv = att.qkv(x).view(b, s, 3, HEADS, DIM // HEADS).permute(2, 0, 3, 1, 4)
    q, k, v = qkv[0], qkv[1], qkv[2]
    scores = (q @ k.transpose(-1, -2)) * att.scale
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else scores + mask
    out = torch.softmax(scores, dim=-1) @ v
    return att.head_concat(out.transpose(1, 2).reshape(b, s, DIM))


@pytest.mark.parametrize("backend", ["sdpa", "math"])
def test_block_mask_equals_separate_attention(backend):
    att = _layer(backend)
    x = torch.randn(2, 12, DIM, dtype=torch.float64)
    y = att(x, _block_mask(5, 7))
    assert torch.allclose(y[:, :5], att(x[:, :5]), atol=1e-10)
    assert torch.allclose(y[:, 5:], att(x[:, 5:]), atol=1e-10)


def test_additive_mask_matches_boolean_and_none_is_neutral():
    att = _layer()
    x = torch.randn(2, 10, DIM, dtype=torch.float64)
    keep = _block_mask(4, 6)
    additive = torch.zeros(10, 10, dtype=torch.float64).masked_fill(~keep, float("-inf"))
    assert torch.allclose(att(x, keep), att(x, additive), atol=1e-12)
    everything = torch.ones(10, 10, dtype=torch.bool)
    assert torch.allclose(att(x, everything), att(x), atol=1e-12)
    assert torch.allclose(att(x, torch.zeros(10, 10, dtype=torch.float64)), att(x), atol=1e-12)


def test_masked_region_is_blind_and_gradients_respect_the_mask():
    att = _layer()
    x = torch.randn(1, 9, DIM, dtype=torch.float64)
    mask = _block_mask(4, 5)
    y0 = att(x, mask)
    x2 = x.clone()
    x2[:, 4:] += torch.randn(1, 5, DIM, dtype=torch.float64)          # change only the second region
    y1 = att(x2, mask)
    assert torch.equal(y0[:, :4], y1[:, :4]), "the first region saw the second through the mask"
    assert not torch.allclose(y0[:, 4:], y1[:, 4:])
    xr = x.clone().requires_grad_(True)
    att(xr, mask)[:, :4].sum().backward()
    assert torch.all(xr.grad[:, 4:] == 0), "gradient leaked through the mask"
    assert torch.any(xr.grad[:, :4] != 0)


@pytest.mark.parametrize("backend", ["sdpa", "math"])
@pytest.mark.parametrize("kind", ["bool", "float"])
def test_arbitrary_mask_matches_explicit_softmax(backend, kind):
    att = _layer(backend, seed=3)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 11, DIM, generator=g, dtype=torch.float64)
    if kind == "bool":
        mask = torch.rand(2, 1, 11, 11, generator=g) > 0.4
        mask |= torch.eye(11, dtype=torch.bool)                     # every query keeps at least itself
    else:
        mask = torch.randn(2, HEADS, 11, 11, generator=g, dtype=torch.float64)
    xr = x.clone().requires_grad_(True)
    y = att(xr, mask)
    xe = x.clone().requires_grad_(True)
    ye = _explicit(att, xe, mask)
    assert torch.allclose(y, ye, atol=1e-10)
    gy = torch.randn(y.shape, generator=g, dtype=torch.float64)
    y.backward(gy)
    ye.backward(gy)
    assert torch.allclose(xr.grad, xe.grad, atol=1e-10)


def _worker_distributed_masks(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col = mesh["row"], mesh["col"]
    g = torch.Generator().manual_seed(9)
    # head-parallel (channel group), no sequence parallelism: windows of 8 tokens, one mask per window
    x = torch.randn(2, 3, 8, DIM, generator=g, dtype=torch.float64)
    masks = {"bool": (torch.rand(3, 1, 8, 8, generator=g) > 0.5) | torch.eye(8, dtype=torch.bool),
             "float": torch.randn(3, 1, 8, 8, generator=g, dtype=torch.float64),
             "block": _block_mask(3, 5)}
    for backend in ("sdpa", "math"):
        att = _layer(backend, qk_norm=True, seed=5)
        for kind, mask in masks.items():
            att.zero_grad()
            xr = x.clone().requires_grad_(True)
            y_ref = att(xr, mask)
            gy = torch.randn(y_ref.shape, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
            y_ref.backward(gy)
            layer = Attention.convert_to_jigsaw(att, mesh, "cpu", ring=False, attn_backend=backend)
            xl = split(x, {3: col}).requires_grad_(True)
            y = layer(xl, mask)
            assert_close(y, split(y_ref.detach(), {3: col}), f"{backend} {kind}: output", 1e-9, 1e-9)
            y.backward(split(gy, {3: col}))
            assert_close(xl.grad, split(xr.grad, {3: col}), f"{backend} {kind}: dx", 1e-9, 1e-9)
    # sequence parallelism refuses a mask instead of ignoring it
    att = _layer("math", seed=6)
    xs = torch.randn(2, 8, DIM, generator=g, dtype=torch.float64)
    mask = torch.ones(8, 8, dtype=torch.bool)
    for kw in ({"ring": True}, {"ring": False, "ulysses": True}):
        layer = Attention.convert_to_jigsaw(att, mesh, "cpu", attn_backend="math", **kw)
        with pytest.raises(ValueError, match=("ring" if kw["ring"] else "ulysses") + " attention does not support"):
            layer(split(xs, {1: row, 2: col}), mask)
        layer(split(xs, {1: row, 2: col}))                            # and still runs without one


def test_masks_with_head_parallel_layers_and_rejection_under_sequence_parallelism():
    run_distributed(_worker_distributed_masks, 4, timeout=300)
