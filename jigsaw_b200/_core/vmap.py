"""Helper for the ``torch.vmap`` rules of the custom autograd Functions (ensemble members as a leading axis).

Every differentiable collective, the halo exchange, the region fetch and the gradient sum carry a ``vmap``
staticmethod: it moves the batched dimension to the front, shifts the dimensions the collective names behind
it and applies the same Function to the whole stack, so one collective moves all members.  Because a rule
re-applies its Function, nested ``vmap`` levels unwind one after the other and work as well
(``tests/test_vmap_cpu.py``).

Reference parity: jigsaw/_core/vmap.py:18-114 (which guards against nesting instead).
"""

from __future__ import annotations

import torch


def to_front(t: torch.Tensor | None, dim: int | None, batch_size: int | None = None) -> torch.Tensor | None:
    """The vmapped dimension moved to the front.  An unbatched tensor is returned as it is, or expanded to
    ``batch_size`` members when that is given."""
    if t is None:
        return None
    if dim is None:
        return t if batch_size is None else t.unsqueeze(0).expand(batch_size, *t.shape)
    return t.movedim(dim, 0)
