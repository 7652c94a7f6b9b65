"""Softmax-type operations along an axis that is cut over a process group.

The maximum and the sum of exponentials are reduced over the group, so every rank normalises its slice with
the global values: ``distributed_softmax`` / ``distributed_log_softmax`` (functions), ``DistributedSoftmax``
(module) and ``distributed_argmax``, which returns global indices and resolves ties to the lowest index.  With
``group=None`` they are the plain ``torch`` operations.  All carry ``vmap`` rules.

Reference parity: jigsaw/modules/activation/__init__.py.
"""

from ..._core.public import set_module
from ._activation import DistributedSoftmax
from ._functional import distributed_argmax, distributed_log_softmax, distributed_softmax

__all__ = ["DistributedSoftmax", "distributed_argmax", "distributed_log_softmax"]

set_module(globals(), __all__)
