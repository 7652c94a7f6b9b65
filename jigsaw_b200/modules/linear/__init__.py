"""Tensor-parallel linear layers and block matrix products."""

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
