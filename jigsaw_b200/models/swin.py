"""Swin Transformer with domain parallelism over a 2-D tile grid (and optional channel split).

The token map ``(B, H / sh, W / sw, C / col)`` is cut into one tile per rank.  A tile holds a
whole number of windows, so window attention, patch merging, the MLP and the norms are local;
only the cyclic shift of the shifted-window blocks moves data between tiles
(``DistributedRoll``: neighbour exchange with wrap-around).  The mask of the shifted windows
follows from the *global* position of each token (tokens that wrapped around the image border
must not attend to the others of their window), so every rank derives it from the position of
its tile.  All weights are replicated over the tile groups (gradients summed in the backward
pass); with a ``col`` axis of size > 1 the linear layers and norms are column-parallel and the
attention heads are split over it.

If a stage's tile is not a multiple of the configured window (deep stages of a finely tiled
map), that stage uses the largest window that divides the tile.

Output: a per-pixel class map ``(B, classes / col, H / patch / sh, W / patch / sw)`` when
``num_classes`` is set (transposed-convolution decoder from the last stage back to the patch
grid), else a correction added to the input image (denoiser).

Reference parity: examples/swin.py:85-283 (window partition, relative position index, shift
mask from the tile position, block, patch merging, model); the class adds configurable
stages, the channel split and the segmentation head of the large benchmark configuration.
"""

from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass

import torch
import torch.utils.checkpoint
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from .. import parallel
from ..modules import DistributedConv2d, DistributedConvTranspose2d, DistributedRoll
from ._layers import TileContext, tile_layer_norm, tile_linear

Mesh = Mapping[str, dist.ProcessGroup]


@dataclass
class SwinConfig:
    image_size: tuple[int, int] = (64, 64)
    in_channels: int = 1
    patch: int = 2
    dims: tuple[int, ...] = (32, 64)
    heads: tuple[int, ...] = (2, 4)
    depths: tuple[int, ...] = (2, 2)
    window: int = 4
    mlp_ratio: int = 4
    num_classes: int | None = None
    dtype: torch.dtype = torch.float32
    recompute_blocks: bool = False      # activation checkpointing: keep only each layer's input, recompute in backward


def window_partition(x: torch.Tensor, ws: int) -> torch.Tensor:
    """``(B, h, w, C)`` -> ``(B, nW, ws * ws, C)`` with windows in row-major order."""
    b, h, w, c = x.shape
    x = x.view(b, h // ws, ws, w // ws, ws, c).permute(0, 1, 3, 2, 4, 5)
    return x.reshape(b, (h // ws) * (w // ws), ws * ws, c)


def window_reverse(x: torch.Tensor, ws: int, h: int, w: int) -> torch.Tensor:
    b, _, _, c = x.shape
    x = x.view(b, h // ws, w // ws, ws, ws, c).permute(0, 1, 3, 2, 4, 5)
    return x.reshape(b, h, w, c)


def relative_position_index(ws: int) -> torch.Tensor:
    """``(ws², ws²)`` index into a ``(2 ws - 1)²`` bias table for every (query, key) offset."""
    pos = torch.stack(torch.meshgrid(torch.arange(ws), torch.arange(ws), indexing="ij")).flatten(1)   # (2, N)
    off = pos[:, :, None] - pos[:, None, :] + (ws - 1)
    return off[0] * (2 * ws - 1) + off[1]


def shifted_window_mask(h: int, w: int, ws: int, shift: int, groups: tuple) -> torch.Tensor:
    """Additive mask ``(nW, ws², ws²)`` of this rank's windows after a global roll by
    ``-shift``: 0 where two tokens come from the same side of the wrap-around seam, -100
    elsewhere."""

    def region(local: int, group: dist.ProcessGroup | None) -> torch.Tensor:
        size, rank = (1, 0) if group is None else (group.size(), group.rank())
        g = rank * local + torch.arange(local)
        total = size * local
        return (g >= total - ws).long() + (g >= total - shift).long()

    label = region(h, groups[0])[:, None] * 3 + region(w, groups[1])[None, :]
    win = window_partition(label[None, :, :, None].float(), ws)[0, :, :, 0]            # (nW, N)
    same = win[:, :, None] == win[:, None, :]
    return torch.zeros(same.shape).masked_fill(~same, -100.0)


class WindowAttention(nn.Module):
    def __init__(self, ctx: TileContext, dim: int, heads: int, ws: int, mask: torch.Tensor | None) -> None:
        super().__init__()
        if heads % ctx.col_size or dim % heads:
            raise ValueError(f"{heads} heads do not split over {ctx.col_size} column ranks / {dim} features")
        self.ws, self.heads, self.head_dim = ws, heads // ctx.col_size, dim // heads
        self.qkv = tile_linear(ctx, dim, 3 * dim)
        self.proj = tile_linear(ctx, dim, dim)
        table = torch.zeros((2 * ws - 1) ** 2, self.heads, device=ctx.device, dtype=ctx.dtype)
        nn.init.trunc_normal_(table, std=0.02)
        self.bias_table = nn.Parameter(table)
        if ctx.live_spatial:
            parallel.mark_replicated(self.bias_table, ctx.live_spatial)
            with torch.no_grad():
                for g in ctx.live_spatial:
                    dist.broadcast(self.bias_table.data, group_src=0, group=g)
        self._col = ctx.col
        self.register_buffer("index", relative_position_index(ws).to(ctx.device), persistent=False)
        self.register_buffer("mask", None if mask is None else mask.to(ctx.device, ctx.dtype), persistent=False)

    def shard_spec(self) -> dict:
        return {"bias_table": ((1, self._col),)}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x``: (B, nW, N, C / col)."""
        b, nw, n, _ = x.shape
        (table,) = parallel.sync_grad(self.bias_table)
        # features are ordered (head, q|k|v, head_dim): a column shard is a whole number of heads
        qkv = self.qkv(x).view(b, nw, n, self.heads, 3, self.head_dim).permute(4, 0, 1, 3, 2, 5)   # (3,B,nW,h,N,d)
        bias = table[self.index.view(-1)].view(n, n, self.heads).permute(2, 0, 1)[None]           # (1,h,N,N)
        if self.mask is not None:
            bias = bias + self.mask[:, None]                                                          # (nW,h,N,N)
        out = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], attn_mask=bias.to(qkv.dtype))
        return self.proj(out.transpose(2, 3).reshape(b, nw, n, self.heads * self.head_dim))


class SwinBlock(nn.Module):
    def __init__(self, ctx: TileContext, dim: int, heads: int, tile: tuple[int, int], ws: int, shift: int, mlp_ratio: int) -> None:
        super().__init__()
        self.tile, self.ws, self.shift = tile, ws, shift
        mask = shifted_window_mask(tile[0], tile[1], ws, shift, ctx.spatial) if shift else None
        self.norm1 = tile_layer_norm(ctx, dim)
        self.attn = WindowAttention(ctx, dim, heads, ws, mask)
        self.norm2 = tile_layer_norm(ctx, dim)
        self.fc1 = tile_linear(ctx, dim, mlp_ratio * dim)
        self.fc2 = tile_linear(ctx, mlp_ratio * dim, dim)
        if shift:
            def roll(s: int) -> nn.Module:
                return DistributedRoll((s, s), (1, 2), (1, 2), ctx.spatial, ctx.device, dtype=ctx.dtype)

            self.shift_in, self.shift_out = roll(-shift), roll(shift)
        else:
            self.shift_in = self.shift_out = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h, w = self.tile
        y = self.norm1(x)
        if self.shift_in is not None:
            y = self.shift_in(y)
        y = window_reverse(self.attn(window_partition(y, self.ws)), self.ws, h, w)
        if self.shift_out is not None:
            y = self.shift_out(y)
        x = x + y
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class PatchMerging(nn.Module):
    """2x2 neighbourhoods (never cut by a tile border) -> one token of twice the width."""

    def __init__(self, ctx: TileContext, dim: int, out_dim: int) -> None:
        super().__init__()
        self.norm = tile_layer_norm(ctx, 4 * dim)
        self.reduce = tile_linear(ctx, 4 * dim, out_dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # features are ordered (channel, neighbour): a column shard keeps whole channels
        parts = torch.stack([x[:, i::2, j::2] for i in (0, 1) for j in (0, 1)], dim=-1)
        return self.reduce(self.norm(parts.flatten(-2)))


def stage_window(tile: tuple[int, int], window: int) -> int:
    """Largest window ``<= window`` that tiles both sides of ``tile``."""
    g = math.gcd(tile[0], tile[1])
    return max(d for d in range(1, min(window, g) + 1) if g % d == 0)


class Swin(nn.Module):
    def __init__(self, mesh: Mesh, device: torch.device | str, cfg: SwinConfig | None = None, row_key: str = "sh",
                 col_key: str = "sw", channel_key: str = "col") -> None:
        super().__init__()
        self.cfg = cfg = cfg or SwinConfig()
        device = torch.device(device)
        sh, sw, col = mesh[row_key], mesh[col_key], mesh[channel_key]
        ctx = TileContext((sh, sw), col, device, cfg.dtype)
        H, W = cfg.image_size
        down = cfg.patch * 2 ** (len(cfg.dims) - 1)
        if H % (down * sh.size()) or W % (down * sw.size()):
            raise ValueError(f"image {H}x{W} must be a multiple of {down} pixels on each of the {sh.size()}x{sw.size()} tiles")
        conv = dict(device=device, spatial_group=(sh, sw), channel_group=col, dtype=cfg.dtype)
        self.embed = DistributedConv2d(cfg.in_channels, cfg.dims[0], kernel_size=cfg.patch, stride=cfg.patch, **conv)
        tile = (H // cfg.patch // sh.size(), W // cfg.patch // sw.size())
        layers: list[nn.Module] = []
        self.windows: list[int] = []
        for i, (dim, heads, depth) in enumerate(zip(cfg.dims, cfg.heads, cfg.depths)):
            ws = stage_window(tile, cfg.window)
            self.windows.append(ws)
            # a window that covers the whole (global) map needs no shift
            whole = ws >= tile[0] * sh.size() and ws >= tile[1] * sw.size()
            for j in range(depth):
                shift = 0 if (j % 2 == 0 or whole or ws < 2) else ws // 2
                layers.append(SwinBlock(ctx, dim, heads, tile, ws, shift, cfg.mlp_ratio))
            if i + 1 < len(cfg.dims):
                layers.append(PatchMerging(ctx, dim, cfg.dims[i + 1]))
                tile = (tile[0] // 2, tile[1] // 2)
        self.layers = nn.Sequential(*layers)
        self.norm = tile_layer_norm(ctx, cfg.dims[-1])
        up = 2 ** (len(cfg.dims) - 1)
        if cfg.num_classes is None:
            self.decode = DistributedConvTranspose2d(cfg.dims[-1], cfg.in_channels, kernel_size=down, stride=down, **conv)
        else:
            self.decode = DistributedConvTranspose2d(cfg.dims[-1], cfg.num_classes, kernel_size=up, stride=up, **conv)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        z = self.embed(x).permute(0, 2, 3, 1).contiguous()           # (B, h, w, C / col)
        if self.cfg.recompute_blocks and torch.is_grad_enabled() and z.requires_grad:
            for layer in self.layers:                                 # same order on every rank: collectives stay matched
                z = torch.utils.checkpoint.checkpoint(layer, z, use_reentrant=False)
        else:
            z = self.layers(z)
        z = self.norm(z).permute(0, 3, 1, 2).contiguous()
        out = self.decode(z)
        return out if self.cfg.num_classes is not None else x + out
