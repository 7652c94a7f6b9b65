"""Activations over sharded dimensions."""

from ..._core.public import set_module
from ._activation import DistributedSoftmax
from ._functional import distributed_argmax, distributed_log_softmax, distributed_softmax

__all__ = ["DistributedSoftmax", "distributed_argmax", "distributed_log_softmax"]

set_module(globals(), __all__)
