"""CPU model of what the thin-channel convolution kernels compute from the packed weight tiles.

The kernels multiply, per output pixel, a row of 48 values gathered from the four-channel padded buffer (nine
taps x four channels, column ``tap * 4 + channel``, padded to 48) with a ``[64][64]`` weight tile.  This test builds
those rows with plain tensor indexing, multiplies them with the tiles ``conv_fused._prep_weights`` produces, and
compares with ``F.conv2d`` / its input gradient: the packing (tap order, channel order, the mirrored taps of the
data gradient, zero padding of unused columns) is pinned without a GPU.
"""

import pytest
import torch
import torch.nn.functional as F

from jigsaw_b200.ops import conv_fused


def _im2col_rows(buf):
    """``buf``: (N, H + 2, W + 2, 4) padded channels-last buffer -> (N, H, W, 48) rows, column tap * 4 + channel."""
    n, hp, wp, _ = buf.shape
    h, w = hp - 2, wp - 2
    taps = [buf[:, dy:dy + h, dx:dx + w, :] for dy in range(3) for dx in range(3)]      # tap = dy * 3 + dx
    rows = torch.cat(taps, dim=-1)                                                       # (N, H, W, 36)
    return F.pad(rows, (0, 12))


def _padded4(x):
    """(N, C <= 4, H, W) -> (N, H + 2, W + 2, 4) with a zero border and zero-filled missing channels."""
    n, c, h, w = x.shape
    buf = torch.zeros(n, h + 2, w + 2, 4, dtype=x.dtype)
    buf[:, 1:-1, 1:-1, :c] = x.permute(0, 2, 3, 1)
    return buf


@pytest.mark.parametrize("cin", [1, 3, 4])
def test_thin_input_forward_tile(cin):
    torch.manual_seed(cin)
    w = torch.randn(64, cin, 3, 3).bfloat16().float()
    b = torch.randn(64)
    x = torch.randn(2, cin, 6, 10).bfloat16().float()
    packed = conv_fused._prep_weights("thin_in", w, b, thin=True)
    tile = packed["w"].float()
    assert tile.shape == (64, 64) and torch.all(tile[:, 36:] == 0), "columns beyond 9 taps x 4 channels must be zero"
    if cin < 4:
        assert torch.all(tile.view(64, 16, 4)[:, :9, cin:] == 0), "missing input channels must be zero"
    rows = _im2col_rows(_padded4(x))                                                     # (N, H, W, 48)
    got = rows @ tile[:, :48].t() + packed["b"]                                          # (N, H, W, 64)
    want = F.conv2d(x, w, b, padding=1).permute(0, 2, 3, 1)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("cout", [1, 3, 4])
def test_thin_output_data_gradient_tile(cout):
    """Data gradient of a 64 -> cout layer = a thin-INPUT convolution of the output gradient (cout channels in the
    four-channel buffer) with mirrored taps: row = input channel of the layer, column = mirrored tap * 4 + output channel."""
    torch.manual_seed(10 + cout)
    w = torch.randn(cout, 64, 3, 3).bfloat16().float()
    gy = torch.randn(2, cout, 6, 10).bfloat16().float()
    packed = conv_fused._prep_weights("thin_out", w, None, thin=True)
    tile = packed["w_dgrad"].float()
    assert tile.shape == (64, 64) and torch.all(tile[:, 36:] == 0)
    rows = _im2col_rows(_padded4(gy))
    got = rows @ tile[:, :48].t()                                                        # (N, H, W, 64)
    x = torch.zeros(2, 64, 6, 10, requires_grad=True)
    F.conv2d(x, w, None, padding=1).backward(gy)
    assert torch.allclose(got, x.grad.permute(0, 2, 3, 1), atol=1e-4, rtol=1e-5)
    # the forward tile of the same layer: 16 output columns, taps first
    fwd = packed["w"].float()
    assert fwd.shape == (3, 3, 16, 64) and torch.all(fwd[:, :, cout:] == 0)
    assert torch.equal(fwd[:, :, :cout], w.permute(2, 3, 0, 1))
    assert packed["b"].shape == (16,) and torch.all(packed["b"] == 0)


def test_mid_layer_tile_and_zero_filled_fallbacks():
    torch.manual_seed(5)
    w = torch.randn(64, 64, 3, 3)
    packed = conv_fused._prep_weights("mid", w, None)
    assert packed["w"].shape == (3, 3, 64, 64) and packed["w"].dtype == torch.bfloat16
    assert torch.equal(packed["w"].float(), w.bfloat16().float().permute(2, 3, 0, 1))      # [dy][dx][co][ci]
    # without the thin kernels (odd tile widths) a thin layer runs zero-filled on the 64-channel kernels
    w3 = torch.randn(64, 3, 3, 3)
    wide = conv_fused._prep_weights("thin_in", w3, None, thin=False)["w"]
    assert wide.shape == (3, 3, 64, 64) and torch.all(wide[..., 3:] == 0)
    w_out = torch.randn(3, 64, 3, 3)
    back = conv_fused._prep_weights("thin_out", w_out, None, thin=False)["w_dgrad"]
    assert back.shape == (3, 3, 64, 64) and torch.all(back[:, :, 3:] == 0)
