"""Tensor-parallel linear layers and block matrix products on a row x column mesh.

``DistributedLinear`` holds one block of the weight per rank (input features cut over rows, output features
over columns) and computes ``x @ W.T + b`` for activations cut the same way; the blocks a rank is missing are
fetched from their owners, on CUDA inside the GEMM kernel's producer warps.  The three ``DistributedMatMul*``
layers are parameter-free products of two block-distributed operands, ``X W``, ``X W^T`` and ``X^T W`` (the
products of two activations inside attention are of this kind); ``MatMulXW`` / ``MatMulXWT`` / ``MatMulXTW``
are their single-device forms, which the converter replaces by the distributed ones.  ``LinearConfig`` records
the grid and the transport (``comm``) that these layers share.

Reference parity: jigsaw/modules/linear/__init__.py (eight public names).
"""

from ..._core.public import set_module
from ._config import LinearConfig
from ._linear import (
    DistributedLinear,
    DistributedMatMulXTW,
    DistributedMatMulXW,
    DistributedMatMulXWT,
    MatMulXTW,
    MatMulXW,
    MatMulXWT,
)

__all__ = [
    "DistributedLinear",
    "DistributedMatMulXTW",
    "DistributedMatMulXW",
    "DistributedMatMulXWT",
    "LinearConfig",
    "MatMulXTW",
    "MatMulXW",
    "MatMulXWT",
]

set_module(globals(), __all__)
