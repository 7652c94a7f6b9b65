"""Vision Transformer with domain and tensor parallelism over a ``(row, col)`` mesh.

Every tensor stays sharded from input to loss::

    image   (B, C / col, H, W / row)     channels over "col", width over "row"
    tokens  (B, N / row, E / col)        sequence over "row", embedding over "col"

    patch embedding   DistributedConv2d, kernel == stride (no halo)
    attention         DistributedAttention: ring or Ulysses over "row", heads over "col"
    MLP               DistributedLinear, weights split over both axes
    norms             DistributedLayerNorm, statistics reduced over "col"
    output            image-to-image (DistributedConvTranspose2d patch recovery, residual)
                      or classification (token mean over "row", class logits over "col")

The position embedding is a fixed 2-D sin/cos function of the *global* patch index, so the
model does not depend on the mesh.

Reference parity: examples/vit.py:63-190 (block, embedding, recovery; 2 blocks of width 64);
this class adds the configurable size, the Ulysses variant and the classification head that
the large benchmark configuration (24 blocks, width 1024, 1000 classes) needs.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass

import torch
import torch.utils.checkpoint
import torch.distributed as dist
from torch import nn

from .._core.collectives import all_reduce_sum
from ..modules import (
    DistributedAttention,
    DistributedConv2d,
    DistributedConvTranspose2d,
    DistributedLayerNorm,
    DistributedLinear,
    RingAttentionConfig,
)
from ..modules.attention import SaveBackward, SendForward

Mesh = Mapping[str, dist.ProcessGroup]


@dataclass
class ViTConfig:
    image_size: tuple[int, int] = (32, 64)
    in_channels: int = 4
    patch: int = 4
    dim: int = 64
    heads: int = 4
    depth: int = 2
    mlp_ratio: int = 4
    num_classes: int | None = None      # None: predict a correction to the input image
    sequence_parallel: str = "ring"     # "ring" | "ulysses"
    attn_backend: str = "sdpa"
    dtype: torch.dtype = torch.float32
    recompute_blocks: bool = False      # activation checkpointing: keep only each block's input, recompute in backward


def sincos_position(dim: int, h_idx: torch.Tensor, w_idx: torch.Tensor) -> torch.Tensor:
    """``(len(h_idx), len(w_idx), dim)`` embedding: the first half encodes the patch row, the
    second half the patch column, each as ``dim / 4`` sines followed by ``dim / 4`` cosines."""
    quarter = dim // 4
    freq = torch.exp(-torch.arange(quarter, dtype=torch.float32) / quarter * torch.log(torch.tensor(10000.0)))

    def encode(idx: torch.Tensor) -> torch.Tensor:
        phase = idx.to(torch.float32)[:, None] * freq[None, :]
        return torch.cat((phase.sin(), phase.cos()), dim=-1)

    eh, ew = encode(h_idx), encode(w_idx)
    grid_h = eh[:, None, :].expand(len(h_idx), len(w_idx), 2 * quarter)
    grid_w = ew[None, :, :].expand(len(h_idx), len(w_idx), 2 * quarter)
    return torch.cat((grid_h, grid_w), dim=-1)


class ViTBlock(nn.Module):
    """Pre-norm block: ``x + attention(norm(x))`` then ``x + mlp(norm(x))``."""

    def __init__(self, cfg: ViTConfig, mesh: Mesh, device: torch.device) -> None:
        super().__init__()
        row, col, model = mesh["row"], mesh["col"], mesh["model"]
        self.norm1 = DistributedLayerNorm(cfg.dim, None, device, row, col, dtype=cfg.dtype)
        self.norm2 = DistributedLayerNorm(cfg.dim, None, device, row, col, dtype=cfg.dtype)
        ring = cfg.sequence_parallel == "ring" and row.size() > 1
        ulysses = cfg.sequence_parallel == "ulysses" and row.size() > 1
        ring_cfg = None
        if ring:
            # keys / values travel (the input slice alone cannot rebuild them under a channel split)
            ring_cfg = RingAttentionConfig(device=device, send_in_forward=SendForward.KV, save_for_backward=SaveBackward.KV,
                                           attn_backend=cfg.attn_backend)
        self.attn = DistributedAttention(
            cfg.dim, cfg.dim, cfg.dim, cfg.heads, None, device, spatial_group=row, channel_group=col, ring=ring,
            ulysses=ulysses, attn_backend=cfg.attn_backend, dtype=cfg.dtype, config=ring_cfg,
        )
        hidden = cfg.mlp_ratio * cfg.dim
        self.fc1 = DistributedLinear(cfg.dim, hidden, device, model, row, col, dtype=cfg.dtype)
        self.act = nn.GELU()
        self.fc2 = DistributedLinear(hidden, cfg.dim, device, model, row, col, dtype=cfg.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.norm1(x))
        return x + self.fc2(self.act(self.fc1(self.norm2(x))))


class ViT(nn.Module):
    def __init__(self, mesh: Mesh, device: torch.device | str, cfg: ViTConfig | None = None) -> None:
        super().__init__()
        self.cfg = cfg = cfg or ViTConfig()
        device = torch.device(device)
        if cfg.sequence_parallel not in ("ring", "ulysses"):
            raise ValueError(f"sequence_parallel must be 'ring' or 'ulysses', got {cfg.sequence_parallel!r}")
        if cfg.dim % 4:
            raise ValueError("dim must be a multiple of 4 for the sin/cos position embedding")
        row, col = mesh["row"], mesh["col"]
        self.row, self.col = row, col
        H, W = cfg.image_size
        if H % cfg.patch or W % (cfg.patch * row.size()):
            raise ValueError(f"image {H}x{W} does not split into {cfg.patch}-pixel patches over {row.size()} row ranks")
        patch = dict(kernel_size=cfg.patch, stride=cfg.patch, device=device, spatial_group=row, channel_group=col,
                     dtype=cfg.dtype)
        self.embed = DistributedConv2d(cfg.in_channels, cfg.dim, **patch)
        self.blocks = nn.ModuleList(ViTBlock(cfg, mesh, device) for _ in range(cfg.depth))
        self.norm = DistributedLayerNorm(cfg.dim, None, device, row, col, dtype=cfg.dtype)
        if cfg.num_classes is None:
            self.recover = DistributedConvTranspose2d(cfg.dim, cfg.in_channels, **patch)
            self.head = None
        else:
            self.recover = None
            # the pooled feature is the same on every row rank; classes are split over "col"
            self.head = DistributedLinear(cfg.dim, cfg.num_classes, device, col, row, col, dtype=cfg.dtype)
        hp, wp, e = H // cfg.patch, W // cfg.patch // row.size(), cfg.dim // col.size()
        pos = sincos_position(cfg.dim, torch.arange(hp), row.rank() * wp + torch.arange(wp))
        pos = pos[..., col.rank() * e : (col.rank() + 1) * e]
        self.register_buffer("pos_embed", pos.to(device=device, dtype=cfg.dtype), persistent=False)
        self.tokens_global = hp * wp * row.size()

    def tokens(self, x: torch.Tensor) -> torch.Tensor:
        """Normalised output tokens ``(B, N / row, E / col)`` of the last block."""
        z = self.embed(x)                                    # (B, E / col, Hp, Wp / row)
        b, e, hp, wp = z.shape
        z = (z.permute(0, 2, 3, 1) + self.pos_embed.to(z.dtype)).reshape(b, hp * wp, e).contiguous()
        for blk in self.blocks:
            if self.cfg.recompute_blocks and torch.is_grad_enabled() and z.requires_grad:
                # every rank recomputes the same block at the same point of its backward pass, so the
                # collectives inside the block stay matched
                z = torch.utils.checkpoint.checkpoint(blk, z, use_reentrant=False)
            else:
                z = blk(z)
        return self.norm(z)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        z = self.tokens(x)
        if self.head is not None:
            pooled = all_reduce_sum(z.sum(dim=1), self.row) / self.tokens_global      # (B, E / col)
            return self.head(pooled)                                                   # (B, classes / col)
        b, _, e = z.shape
        hp = self.cfg.image_size[0] // self.cfg.patch
        z = z.reshape(b, hp, -1, e).permute(0, 3, 1, 2).contiguous()
        return x + self.recover(z)
