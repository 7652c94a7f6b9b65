"""3-D encoder-decoder with domain parallelism over the two trailing spatial axes.

A volume ``(B, C, D, H / sh, W / sw)`` goes down through strided ``DistributedConv3d`` layers
(kernel 3, stride 2, padding 1: one halo plane from the lower neighbour on each split axis)
and back up through ``DistributedConvTranspose3d`` layers (kernel 4, stride 2, padding 1: the
outputs overlap the tile border by one plane, which exercises the halo *reduce*), with
``DistributedGroupNorm`` (statistics over the tile groups) and GELU after each layer but the
last.  The decoder adds the encoder feature of the same resolution (skip connections).

Reference parity: the reference ships the 3-D layers (convolution/_conv/conv.py:25-33,
_conv_transpose/conv_transpose.py, normalization/_distributed_group_norm.py) but no 3-D
model; this is the model of its 3-D benchmark configuration (channels 1-32-64-128).
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass

import torch
import torch.utils.checkpoint
import torch.distributed as dist
from torch import nn

from ..modules import DistributedConv3d, DistributedConvTranspose3d, DistributedGroupNorm

Mesh = Mapping[str, dist.ProcessGroup]


@dataclass
class UNet3dConfig:
    in_channels: int = 1
    out_channels: int = 1
    widths: tuple[int, ...] = (32, 64, 128)
    norm_groups: int = 8
    skip: bool = True
    dtype: torch.dtype = torch.float32
    recompute_stages: bool = False      # activation checkpointing: keep each stage's input, recompute conv + norm + GELU in backward


class UNet3d(nn.Module):
    def __init__(self, mesh: Mesh, device: torch.device | str, cfg: UNet3dConfig | None = None, row_key: str = "sh",
                 col_key: str = "sw", channel_key: str = "col") -> None:
        super().__init__()
        self.cfg = cfg = cfg or UNet3dConfig()
        device = torch.device(device)
        spatial = (None, mesh[row_key], mesh[col_key])
        col = mesh[channel_key]
        kw = dict(device=device, spatial_group=spatial, channel_group=col, dtype=cfg.dtype)

        def norm(ch: int) -> nn.Module:
            return DistributedGroupNorm(cfg.norm_groups, ch, device, channel_group=col, dtype=cfg.dtype, spatial_group=spatial)

        chans = (cfg.in_channels, *cfg.widths)
        self.down = nn.ModuleList(DistributedConv3d(chans[i], chans[i + 1], 3, stride=2, padding=1, **kw)
                                  for i in range(len(cfg.widths)))
        self.down_norm = nn.ModuleList(norm(c) for c in cfg.widths)
        ups = (*reversed(cfg.widths[:-1]), cfg.out_channels)
        ins = (cfg.widths[-1], *ups[:-1])
        self.up = nn.ModuleList(DistributedConvTranspose3d(ins[i], ups[i], 4, stride=2, padding=1, **kw)
                                for i in range(len(ups)))
        self.up_norm = nn.ModuleList(norm(c) for c in ups[:-1])
        self.act = nn.GELU()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        feats = []
        recompute = self.cfg.recompute_stages and torch.is_grad_enabled()
        for conv, norm in zip(self.down, self.down_norm):
            stage = lambda t, conv=conv, norm=norm: self.act(norm(conv(t)))  # noqa: E731
            # the first stage's input needs no gradient, which the non-reentrant form handles
            x = torch.utils.checkpoint.checkpoint(stage, x, use_reentrant=False) if recompute else stage(x)
            feats.append(x)
        feats.pop()
        for i, conv in enumerate(self.up):
            x = conv(x)
            if i < len(self.up_norm):
                x = self.act(self.up_norm[i](x))
                if self.cfg.skip:
                    x = x + feats.pop()
        return x
