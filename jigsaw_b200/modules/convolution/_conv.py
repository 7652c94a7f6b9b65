"""Domain- and channel-parallel convolutions and transposed convolutions (1-, 2-, 3-D).

A layer takes GLOBAL channel counts plus process groups and works on the local tile:
``x`` is ``(N, Cin / G, *spatial / tiles)`` (or unbatched), the weight is sharded over the
output channels of the channel group and replicated (marked, broadcast at construction)
over every split spatial group.

Forward, as a composition of differentiable pieces (autograd derives the distributed
backward: data gradient + halo scatter-add + channel reduce-scatter, weight gradient):

    channels : all-gather of the input channels, or a ring of partial convolutions that
               overlaps each hop with the previous block's convolution
    halo     : per split axis, ``span_gather`` (conv) before / ``span_reduce`` (transposed
               conv) after the local primitive, which runs with padding 0 on split axes
    patchify : ``kernel == stride``, padding 0, dilation 1 tiles the domain, no halo

On CUDA, 3x3 / stride 1 / padding 1 layers with 64 input channels in bf16 take the fused
sm_100a path (``jigsaw_b200.ops.conv_fused``): implicit GEMM on tcgen05 with the halo
written straight into the neighbours' buffers by the producing kernel.

Reference parity: jigsaw/modules/convolution/_conv/base.py:28-688,
_conv/distributed.py:39-396, _conv/channel_comm.py:31-220, _conv_transpose/base.py,
_conv_transpose/distributed.py:23-446, _conv_transpose/channel_comm.py:39-251.
"""

from __future__ import annotations

import math
from collections.abc import Sequence
from typing import Any

import torch
import torch.distributed as dist

from ... import init, parallel
from ..._core.collectives import all_gather_cat, ring_pass
from ..._core.comm import CommOp, resolve_comm_op
from ..._core.config import check_config
from ..._core.placement import gather_dim
from ..._core.shard_repr import shard_repr
from ._args import layer_key, ntuple, resolve_conv_groups, resolve_padding, spatial_groups_tuple
from ._config import ConvNdConfig, ConvTransposeNdConfig
from ._halo import conv_axis_plan, conv_transpose_axis_plan, span_gather, span_reduce

_TORCH_CONV = {1: torch.nn.Conv1d, 2: torch.nn.Conv2d, 3: torch.nn.Conv3d}
_TORCH_CONV_T = {1: torch.nn.ConvTranspose1d, 2: torch.nn.ConvTranspose2d, 3: torch.nn.ConvTranspose3d}


class _DistributedConvBase(torch.nn.Module):
    _n_spatial = 2
    _transposed = False

    def __init__(
        self,
        in_channels: int,
        out_channels: int,
        kernel_size: int | tuple[int, ...],
        device: torch.device | str,
        spatial_group: "dist.ProcessGroup | Sequence[dist.ProcessGroup | None]",
        channel_group: dist.ProcessGroup,
        stride: int | tuple[int, ...] = 1,
        padding: int | str | tuple[int, ...] = (0,),
        dilation: int | tuple[int, ...] = 1,
        groups: int = 1,
        bias: bool = True,
        dtype: torch.dtype = torch.float32,
        channel_comm: CommOp | str = "auto",
        config: Any = None,
        output_padding: int | tuple[int, ...] = 0,
    ) -> None:
        super().__init__()
        n = self._n_spatial
        if self._transposed:
            if isinstance(padding, str):
                raise NotImplementedError(f"transposed convolutions do not take string padding ({padding!r}): give the padding of each axis as a number")
            if any(o != 0 for o in ntuple(output_padding, n)):
                raise NotImplementedError("output_padding is not supported by distributed transposed convolutions")
        self.groups = groups
        G = channel_group.size()
        self._channel_local, self._groups_local = resolve_conv_groups(groups, in_channels, out_channels, G)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.local_out_channels = out_channels // G
        self.local_in_channels = in_channels // G
        self.kernel_size = ntuple(kernel_size, n)
        self.stride = ntuple(stride, n)
        self.dilation = ntuple(dilation, n)
        self.padding = resolve_padding(padding, self.kernel_size, self.stride, self.dilation)
        self.channel_comm = channel_comm
        self.spatial_groups = spatial_groups_tuple(spatial_group, n)
        self.channel_group = channel_group
        self.device = torch.device(device)
        self.dtype = dtype
        self._check_padding(self.spatial_groups, self._channel_local)
        self._spatial_sync_groups = [g for g in self.spatial_groups if g is not None and g.size() > 1]
        self._set_shapes()
        self.weight = torch.nn.Parameter(torch.zeros(self._local_weight_shape(), device=self.device, dtype=dtype))
        self.bias = (
            torch.nn.Parameter(torch.zeros(self.local_out_channels, device=self.device, dtype=dtype)) if bias else None
        )
        self.reset_parameters()
        key = layer_key(channel_group, self.bias, self.kernel_size, self.stride, groups)
        if config is not None:
            check_config(config, key)
        cfg_cls = ConvTransposeNdConfig if self._transposed else ConvNdConfig
        self.config = config or cfg_cls(
            channel_group, self.bias, self.kernel_size, self.stride, self.device, channel_comm, groups
        )
        self._halo_comm = resolve_comm_op("auto", self.device)
        self._mark_and_broadcast()
        self._plans: dict[tuple, Any] = {}
        self.fused_activation: str | None = None   # set by fusing containers (e.g. "gelu")

    # ------------------------------------------------------------------ shapes / init
    def _set_shapes(self) -> None:
        if self._transposed:
            # torch layout (Cin, Cout / groups, *k); sharded on dim 1 (output channels), or on
            # dim 0 (input channels) when every rank owns whole convolution groups.
            self.global_weight_shape = (self.in_channels, self.out_channels // self.groups, *self.kernel_size)
        else:
            self.global_weight_shape = (self.out_channels, self.in_channels // self.groups, *self.kernel_size)
        self.global_bias_shape = (self.out_channels,)

    @property
    def _weight_shard_dim(self) -> int:
        if not self._transposed:
            return 0
        return 0 if (self._channel_local and self.groups > 1) else 1

    def _local_weight_shape(self) -> tuple[int, ...]:
        shape = list(self.global_weight_shape)
        shape[self._weight_shard_dim] //= self.channel_group.size()
        return tuple(shape)

    def reset_parameters(self) -> None:
        """Same distributions as the torch layer: fans come from the global weight shape."""
        init.kaiming_uniform_(self.weight, a=math.sqrt(5), global_shape=self.global_weight_shape)
        if self.bias is not None:
            shape = self.global_weight_shape
            fan_in = shape[1] * math.prod(shape[2:])
            bound = 1.0 / math.sqrt(fan_in) if fan_in > 0 else 0.0
            init.uniform_(self.bias, -bound, bound)

    def _mark_and_broadcast(self) -> None:
        for p in self.parameters():
            if not parallel.replica_groups(p):
                parallel.mark_replicated(p, self._spatial_sync_groups)
        with torch.no_grad():
            for p in self.parameters():
                for g in reversed(self._spatial_sync_groups):
                    dist.broadcast(p.data, group_src=0, group=g)

    def _check_padding(self, spatial_groups: tuple, channel_local: bool) -> None:
        split = any(g is not None and g.size() > 1 for g in spatial_groups)
        if self.padding == "same" and (split or not channel_local):
            raise NotImplementedError(
                f"padding='same' with kernel_size={self.kernel_size} and dilation={self.dilation} pads "
                "asymmetrically, which is only supported without a spatial split and with whole "
                "conv-groups per channel rank; use an odd kernel_size or explicit padding."
            )

    # ------------------------------------------------------------------ introspection
    @property
    def spatial_world_size(self) -> int:
        """Number of spatial ranks the parameters are replicated over."""
        return math.prod(g.size() for g in self._spatial_sync_groups)

    def shard_spec(self) -> dict:
        """Which dimension of which parameter is cut over which group (sharded checkpoints)."""
        return {"weight": ((self._weight_shard_dim, self.channel_group),), "bias": ((0, self.channel_group),)}

    def get_parameter_count(self) -> int:
        """Global (unsharded) number of weight and bias elements; no communication."""
        nb = math.prod(self.global_bias_shape) if self.bias is not None else 0
        return nb + math.prod(self.global_weight_shape)

    def extra_repr(self) -> str:
        s = f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}"
        if self.padding != (0,) * self._n_spatial:
            s += f", padding={self.padding}"
        if self.dilation != (1,) * self._n_spatial:
            s += f", dilation={self.dilation}"
        if self.groups != 1:
            s += f", groups={self.groups}"
        if self.bias is None:
            s += ", bias=False"
        return s + ", " + shard_repr(spatial=self.spatial_groups, channel=self.channel_group)

    # ------------------------------------------------------------------ conversion / resharding
    @classmethod
    def convert_to_jigsaw(
        cls,
        model: torch.nn.modules.conv._ConvNd,
        process_mesh_dict: dict,
        device: torch.device | str,
        row_kw: str = "row",
        col_kw: str = "col",
        model_kw: str = "model",
        **kwargs: Any,
    ) -> "_DistributedConvBase":
        """Build the distributed layer from a torch layer and slice its parameters.

        The spatial group is ``process_mesh_dict[row_kw]`` (splits the last axis) unless
        ``spatial_group=`` is passed; channels are sharded over ``process_mesh_dict[col_kw]``.
        """
        if model.padding_mode != "zeros":
            raise NotImplementedError(
                f"padding_mode={model.padding_mode!r} is not supported; distributed convolutions pad with zeros only."
            )
        extra = {}
        if cls._transposed:
            extra["output_padding"] = model.output_padding
        layer = cls(
            in_channels=model.in_channels,
            out_channels=model.out_channels,
            kernel_size=model.kernel_size,
            stride=model.stride,
            padding=model.padding,
            dilation=model.dilation,
            groups=model.groups,
            bias=model.bias is not None,
            spatial_group=kwargs.get("spatial_group", process_mesh_dict[row_kw]),
            channel_group=process_mesh_dict[col_kw],
            device=device,
            dtype=model.weight.dtype,
            channel_comm=kwargs.get("channel_comm", kwargs.get("comm", "auto")),
            **extra,
        )
        layer._load_global(model.weight.data, None if model.bias is None else model.bias.data)
        return layer

    def _load_global(self, weight: torch.Tensor, bias: torch.Tensor | None) -> None:
        G, r = self.channel_group.size(), self.channel_group.rank()
        d = self._weight_shard_dim
        block = weight.shape[d] // G
        with torch.no_grad():
            self.weight.data = weight.narrow(d, r * block, block).clone().to(self.device).contiguous()
            if bias is not None and self.bias is not None:
                b = bias.shape[0] // G
                self.bias.data = bias[r * b : (r + 1) * b].clone().to(self.device)

    def merge_weights(self, process_mesh_dict: dict, col_kw: str = "col") -> tuple[torch.Tensor, torch.Tensor | None]:
        """All-gather the channel shards into the global weight and bias (collective)."""
        g = process_mesh_dict[col_kw]
        with torch.no_grad():
            w = gather_dim(self.weight.detach(), g, self._weight_shard_dim)
            b = gather_dim(self.bias.detach(), g, 0) if self.bias is not None else None
        return w, b

    def convert_to_torch(
        self, process_mesh_dict: dict, row_kw: str = "row", col_kw: str = "col", model_kw: str = "model"
    ) -> torch.nn.modules.conv._ConvNd:
        """Merge the shards into a plain ``torch.nn`` layer (collective)."""
        w, b = self.merge_weights(process_mesh_dict, col_kw)
        cls = (_TORCH_CONV_T if self._transposed else _TORCH_CONV)[self._n_spatial]
        layer = cls(
            in_channels=self.in_channels,
            out_channels=self.out_channels,
            kernel_size=self.kernel_size,
            stride=self.stride,
            padding=self.padding,
            dilation=self.dilation,
            groups=self.groups,
            bias=b is not None,
            padding_mode="zeros",
        )
        layer.weight.data = w
        if b is not None:
            layer.bias.data = b
        return layer

    def reshard_parameters(
        self,
        from_process_mesh_dict: dict,
        to_process_mesh_dict: dict,
        pm_row_key: str = "row",
        pm_col_key: str = "col",
        pm_model_key: str = "model",
    ) -> None:
        """Move the parameters from one mesh to another: merge over the old channel group,
        re-slice for the new one, rebind the groups and re-mark / re-broadcast the replicas."""
        new_channel = to_process_mesh_dict[pm_col_key]
        new_spatial = spatial_groups_tuple(to_process_mesh_dict[pm_row_key], self._n_spatial)
        local, _ = resolve_conv_groups(self.groups, self.in_channels, self.out_channels, new_channel.size())
        self._check_padding(new_spatial, local)
        w, b = self.merge_weights(from_process_mesh_dict, pm_col_key)
        self.channel_group = new_channel
        self.spatial_groups = new_spatial
        self._spatial_sync_groups = [g for g in new_spatial if g is not None and g.size() > 1]
        self._channel_local, self._groups_local = resolve_conv_groups(
            self.groups, self.in_channels, self.out_channels, new_channel.size()
        )
        self.local_out_channels = self.out_channels // new_channel.size()
        self.local_in_channels = self.in_channels // new_channel.size()
        has_bias = self.bias is not None
        self.weight = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=w.dtype))
        if has_bias:
            self.bias = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=w.dtype))
        self._load_global(w, b)
        self.config = type(self.config)(
            new_channel, self.bias, self.kernel_size, self.stride, self.device, self.config.channel_comm, self.groups
        )
        self._plans.clear()
        self._mark_and_broadcast()

    # ------------------------------------------------------------------ forward
    def _is_patchify(self) -> bool:
        pad0 = self.padding == (0,) * self._n_spatial
        return self.kernel_size == self.stride and pad0 and all(d == 1 for d in self.dilation)

    def _needs_halo(self) -> bool:
        return bool(self._spatial_sync_groups) and not self._is_patchify()

    def _split_axes(self) -> list[tuple[int, dist.ProcessGroup]]:
        """``(axis index, group)`` of every split spatial axis, outermost first."""
        return [(i, g) for i, g in enumerate(self.spatial_groups) if g is not None and g.size() > 1]

    def _local_padding(self) -> Any:
        if isinstance(self.padding, str):
            return self.padding
        if not self._needs_halo():
            return self.padding
        split = {i for i, _ in self._split_axes()}
        return tuple(0 if i in split else p for i, p in enumerate(self.padding))

    def _primitive(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
        fn = self.config.native_fn
        if x.is_cuda and not self._transposed and self._is_patchify() and self._groups_local == 1:
            from ...ops import conv_fused

            # patch embedding (kernel == stride): one patch-gather copy and one tcgen05 GEMM with the bias in its epilogue
            y = conv_fused.maybe_fused_patch_embed(x, w, b, self.kernel_size)
            if y is not None:
                return y
        if self._transposed:
            return fn(x, w, b, self.stride, self._local_padding(), 0, self._groups_local, self.dilation)
        return fn(x, w, b, self.stride, self._local_padding(), self.dilation, self._groups_local)

    def _plan(self, axis: int, group: dist.ProcessGroup, n_local: int) -> Any:
        key = (axis, id(group), n_local)
        if key not in self._plans:
            dim = axis - self._n_spatial
            args = (dim, group, n_local, self.kernel_size[axis], self.stride[axis], self.padding[axis],
                    self.dilation[axis], self._halo_comm)
            if self._transposed:
                self._plans[key] = conv_transpose_axis_plan(*args)
            else:
                self._plans[key] = conv_axis_plan(*args)[0]
        return self._plans[key]

    def _channel_conv(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
        """Local primitive over the full input channels (all-gather or streaming ring)."""
        G = self.channel_group.size()
        if G == 1 or self._channel_local:
            return self._primitive(x, w, b)
        ring = self.config.ring_comm
        cdim = 1
        if ring is None:
            return self._primitive(all_gather_cat(x, self.channel_group, cdim), w, b)
        # Ring: block (r + step) of the input channels is convolved with the matching slice
        # of the weight while the next block is already travelling.
        r = self.channel_group.rank()
        width = x.shape[cdim]
        wdim = 0 if self._transposed else 1
        out = None
        block = x
        for step in range(G):
            src = (r + step) % G
            nxt = ring_pass(block, self.channel_group, -1, ring) if step + 1 < G else None
            ws = w.narrow(wdim, src * width, width)
            part = self._primitive(block, ws, b if step == 0 else None)
            out = part if out is None else out + part
            block = nxt
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Local tile in, local tile out; see the module docstring for the shapes."""
        n = self._n_spatial
        if x.dim() not in (n + 1, n + 2):
            raise ValueError(f"expected {n + 1}D (unbatched) or {n + 2}D (batched) input, got {x.dim()}D")
        unbatched = x.dim() == n + 1
        if unbatched:
            x = x.unsqueeze(0)
        lazy, x = self._try_fused(x)
        if lazy is not None:
            return lazy            # computed when something other than GELU / the next eligible layer touches it
        w, b = parallel.sync_grad(self.weight, self.bias)
        if not self._needs_halo():
            if self._is_patchify() and not self._transposed:
                for i, g in self._split_axes():
                    if x.shape[i - n] % self.stride[i]:
                        raise ValueError(
                            f"kernel_size == stride: the local size {x.shape[i - n]} of split axis {i} must be "
                            f"a multiple of the stride {self.stride[i]}"
                        )
            y = self._channel_conv(x, w, b)
        elif self._transposed:
            y = self._channel_conv(x, w, None)
            for i, g in reversed(self._split_axes()):
                y = span_reduce(y, self._plan(i, g, x.shape[i - n]))
            if b is not None:
                y = y + b.view(1, -1, *([1] * n)).to(y.dtype)
        else:
            try:
                for i, g in self._split_axes():
                    x = span_gather(x, self._plan(i, g, x.shape[i - n]))
            except ValueError as err:
                raise NotImplementedError(str(err)) from err
            y = self._channel_conv(x, w, b)
        return y.squeeze(0) if unbatched else y

    def _try_fused(self, x: torch.Tensor) -> tuple[torch.Tensor | None, torch.Tensor]:
        """``(pending fused result or None, input to continue with)``; the input comes back computed if it
        arrived as a pending fused chain that this layer cannot join."""
        if x.is_cuda:
            from ...ops.lazy_chain import materialize

            x = materialize(x)
        return None, x


class _DistributedConvNd(_DistributedConvBase):
    _transposed = False

    def _try_fused(self, x: torch.Tensor) -> tuple[torch.Tensor | None, torch.Tensor]:
        if not x.is_cuda:
            return None, x
        from ...ops import _lib, conv_fused

        if _lib._any_batched((x, self.weight)):     # under torch.vmap: the kernels have no batching rules
            return None, x

        if self._n_spatial != 2 or x.dim() != 4 or self._is_patchify():
            from ...ops.lazy_chain import materialize

            return None, materialize(x)          # patch embedding has its own fused path (see _primitive)
        return conv_fused.fused_or_lazy_conv2d(self, x)


class _DistributedConvTransposeNd(_DistributedConvBase):
    _transposed = True


class DistributedConv1d(_DistributedConvNd):
    """``torch.nn.Conv1d`` over a length split across ``spatial_group``."""

    _n_spatial = 1


class DistributedConv2d(_DistributedConvNd):
    """``torch.nn.Conv2d`` over an image tiled across up to two spatial groups."""

    _n_spatial = 2


class DistributedConv3d(_DistributedConvNd):
    """``torch.nn.Conv3d`` over a volume tiled across up to three spatial groups."""

    _n_spatial = 3


class DistributedConvTranspose1d(_DistributedConvTransposeNd):
    """``torch.nn.ConvTranspose1d`` with an output-side halo reduce."""

    _n_spatial = 1


class DistributedConvTranspose2d(_DistributedConvTransposeNd):
    """``torch.nn.ConvTranspose2d`` with an output-side halo reduce."""

    _n_spatial = 2


class DistributedConvTranspose3d(_DistributedConvTransposeNd):
    """``torch.nn.ConvTranspose3d`` with an output-side halo reduce."""

    _n_spatial = 3
