"""Domain-parallel CNN: a stack of 3x3 ``DistributedConv2d`` layers with GELU between them.

The image is tiled over the ``(sh, sw)`` axes of the mesh, every rank holds all weights
(replicated, marked, gradients summed over the spatial groups).  On CUDA under bf16 autocast
an eligible stack runs as ONE fused chain (``jigsaw_b200.ops.conv_fused``): each layer's
epilogue applies bias + GELU, writes the next layer's padded input and stores its edge pixels
into the neighbouring ranks' buffers.  Elsewhere (CPU / gloo, fp32, other shapes) the layers
run one by one on the ``torch.distributed`` path with identical results.

Reference parity: the CNN of examples/domain_parallel.py:47-88 built from
jigsaw.modules.DistributedConv2d and nn.GELU; here scaled to the benchmark configuration
(8 layers, 64 channels, 3 input / output channels).
"""

from __future__ import annotations

from collections.abc import Mapping

import torch
import torch.distributed as dist
from torch import nn

from .. import parallel
from ..modules import DistributedConv2d


class DomainCNN(nn.Module):
    """``depth`` convolutions ``in_ch -> width -> ... -> width -> out_ch`` (k3, p1) with GELU between."""

    def __init__(
        self,
        mesh: Mapping[str, dist.ProcessGroup],
        device: torch.device | str,
        in_channels: int = 3,
        out_channels: int = 3,
        width: int = 64,
        depth: int = 8,
        row_key: str = "sh",
        col_key: str = "sw",
        channel_key: str = "col",
        dtype: torch.dtype = torch.float32,
        fuse: bool = True,
    ) -> None:
        super().__init__()
        if depth < 2:
            raise ValueError("depth must be at least 2")
        self.spatial = (mesh.get(row_key), mesh[col_key])
        chans = [in_channels] + [width] * (depth - 1) + [out_channels]
        self.convs = nn.ModuleList(
            DistributedConv2d(chans[i], chans[i + 1], 3, device, self.spatial, mesh[channel_key], padding=1, dtype=dtype)
            for i in range(depth)
        )
        self.act = nn.GELU()
        self.fuse = fuse

    def _fused(self, x: torch.Tensor) -> torch.Tensor | None:
        if not (self.fuse and x.is_cuda):
            return None
        from ..ops import _lib, conv_fused

        kinds = conv_fused.chain_kinds([(c.in_channels, c.out_channels) for c in self.convs])
        if x.requires_grad or kinds is None or not all(conv_fused.layer_is_eligible(c, x) for c in self.convs):
            _lib.decline("the stack needs bf16 numerics, 3x3 / stride 1 / padding 1 layers and 64 inner channels")
            _lib.record("conv_chain", False)          # raises under strict dispatch
            return None
        _lib.record("conv_chain", True)
        raw = [t for c in self.convs for t in (c.weight, c.bias)]
        geom = conv_fused.geometry_for(x, *self.spatial)
        acts = [True] * (len(self.convs) - 1) + [False]
        ranks = parallel.overlapped_sum_plan(raw)
        if ranks is not None:
            # every layer's gradients are summed over the tile ranks by the chain itself, on a side stream,
            # while the rest of its backward pass runs
            return conv_fused.conv_chain(x, geom, kinds, acts, raw[0::2], raw[1::2], reduce_ranks=ranks)
        # one call: all replicated gradients travel in a single flattened all-reduce per group
        params = list(parallel.sync_grad(*raw))
        return conv_fused.conv_chain(x, geom, kinds, acts, params[0::2], params[1::2])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = self._fused(x)
        if out is not None:
            return out
        for i, conv in enumerate(self.convs):
            x = conv(x)
            if i + 1 < len(self.convs):
                x = self.act(x)
        return x
