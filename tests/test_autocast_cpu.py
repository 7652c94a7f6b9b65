"""Autocast contracts of the distributed layers on CPU ranks (``torch.autocast("cpu", bf16)``):

* the matmul family (linear with bias, convolutions, attention incl. ring) runs forward in the autocast
  dtype and returns gradients in the dtype of the inputs / parameters;
* LayerNorm and softmax follow the fp32-list rule: computed and emitted in fp32 under autocast;
* nothing goes non-finite and every result tracks the run without autocast.

Reference behaviours covered: tests/test_autocast.py:89-133 (linear), :135-260 (attention, ring attention),
:262-359 (LayerNorm with and without parameters, softmax), :361-432 (convolution).
"""

import contextlib

import pytest
import torch

from dist_utils import assert_close, run_distributed

TOL = 3e-2


def _run(model, x, autocast, seed=0, half=torch.bfloat16):
    model.zero_grad(set_to_none=True)
    x = x.clone().detach().requires_grad_(True)
    ctx = torch.autocast("cpu", dtype=half) if autocast else contextlib.nullcontext()
    with ctx:
        y = model(x)
    g = torch.randn(y.shape, generator=torch.Generator().manual_seed(seed)).to(y.dtype)
    y.backward(g)                                    # backward outside the autocast region, as training does
    assert x.grad is not None
    return y.detach(), x.grad.detach()


def _check(name, model, x, out_dtype, tol=TOL, half=torch.bfloat16):
    y, dx = _run(model, x, True, half=half)
    y_ref, dx_ref = _run(model, x, False)
    assert y.dtype == out_dtype, f"{name}: forward output is {y.dtype}, expected {out_dtype}"
    assert dx.dtype == x.dtype, f"{name}: input gradient is {dx.dtype}, not the input dtype {x.dtype}"
    assert torch.isfinite(y).all() and torch.isfinite(dx).all(), f"{name}: non-finite values"
    for p in model.parameters():
        assert p.grad is None or p.grad.dtype == p.dtype, f"{name}: parameter gradient in {p.grad.dtype}"
    scale = float(y_ref.abs().max()) + 1e-6
    assert_close(y.to(y_ref.dtype), y_ref, f"{name}: output", tol, tol * scale)
    assert_close(dx, dx_ref, f"{name}: input gradient", tol, tol * (float(dx_ref.abs().max()) + 1e-6))


def _worker_autocast(rank, world, half):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import RingAttentionConfig

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    M = jb.modules
    torch.manual_seed(rank)
    for bias in (False, True):
        layer = M.DistributedLinear(10, 20, "cpu", model, row, col, bias=bias)
        _check(f"linear bias={bias}", layer, torch.randn(1, 10, 5), half, half=half)
    conv = M.DistributedConv2d(4, 8, 3, "cpu", row, col, padding=1)
    _check("conv2d", conv, torch.randn(2, 2, 6, 4), half, half=half)
    convt = M.DistributedConvTranspose2d(4, 8, 2, "cpu", row, col, stride=2)
    _check("conv transpose 2d", convt, torch.randn(2, 2, 6, 4), half, half=half)
    att = M.DistributedAttention(16, 16, 16, 4, col.rank(), "cpu", row, col, attn_backend="math")
    _check("attention", att, torch.randn(2, 8, 8), half, tol=6e-2, half=half)
    cfg = RingAttentionConfig(device="cpu", attn_backend="math", send_in_forward="kv")
    ring = M.DistributedAttention(16, 16, 16, 4, col.rank(), "cpu", row, col, ring=True, attn_backend="math", config=cfg)
    _check("ring attention", ring, torch.randn(2, 4, 8), half, tol=6e-2, half=half)
    # fp32-list layers: fp32 out under autocast, also when fed bf16
    ln = M.DistributedLayerNorm(16, model.rank(), "cpu", row, col)
    _check("layer norm", ln, torch.randn(2, 4, 8), torch.float32, half=half)
    ln0 = M.DistributedLayerNorm(16, model.rank(), "cpu", row, col, elementwise_affine=False)
    _check("layer norm without parameters", ln0, torch.randn(2, 4, 8), torch.float32, half=half)
    sm = M.DistributedSoftmax(col, dim=-1)
    _check("softmax", sm, torch.randn(2, 4, 8), torch.float32, half=half)
    with torch.autocast("cpu", dtype=half):
        assert ln(torch.randn(2, 4, 8).to(half)).dtype == torch.float32
        assert sm(torch.randn(2, 4, 8).to(half)).dtype == torch.float32


@pytest.mark.parametrize("half", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_autocast_contracts_on_four_ranks(half):
    run_distributed(_worker_autocast, 4, half, timeout=300)
