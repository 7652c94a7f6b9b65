"""Per-layer configuration objects of the convolution layers.

A config resolves the channel-communication strategy and the local primitive once, at
construction, and records the layer properties it was built for so that a config passed
to a different layer is rejected.

Reference parity: jigsaw/modules/convolution/_conv/config.py:32-120,
_conv_transpose/config.py:22-116, _common/config.py:9-43.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..._core.comm import CommOp
from ._args import layer_key, resolve_channel_comm

_CONV = (F.conv1d, F.conv2d, F.conv3d)
_CONV_T = (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)


class _ConvConfigBase:
    transposed = False

    def __init__(
        self,
        channel_group: dist.ProcessGroup,
        bias: torch.Tensor | None,
        kernel_size: tuple[int, ...],
        stride: tuple[int, ...],
        device: torch.device | str,
        channel_comm: CommOp | str = "auto",
        groups: int = 1,
    ) -> None:
        self.n_spatial = len(kernel_size)
        self.device = torch.device(device)
        self.channel_comm = resolve_channel_comm(channel_comm, self.device)
        self.groups = groups
        self._layer_key = layer_key(channel_group, bias, kernel_size, stride, groups)
        G = channel_group.size()
        self.channel_local = groups % G == 0
        self.groups_local = groups // G if self.channel_local else 1
        self.patchify = tuple(kernel_size) == tuple(stride)
        self.native_fn = (_CONV_T if self.transposed else _CONV)[self.n_spatial - 1]
        self.vmapped = False

    def for_vmap(self) -> "_ConvConfigBase":
        """Copy whose local primitive is vmapped over a leading members axis (ensembles)."""
        import copy

        other = copy.copy(self)
        other.native_fn = torch.vmap(self.native_fn)
        other.vmapped = True
        return other

    @property
    def ring_comm(self) -> CommOp | None:
        """Transport of the streaming channel ring, or ``None`` for the all-gather strategy."""
        return None if self.channel_comm == "all_gather" else CommOp(self.channel_comm)


class ConvNdConfig(_ConvConfigBase):
    """Kernel selection of ``DistributedConv{1,2,3}d``."""

    transposed = False


class ConvTransposeNdConfig(_ConvConfigBase):
    """Kernel selection of ``DistributedConvTranspose{1,2,3}d``."""

    transposed = True
