"""``DistributedLinear`` and the ``(Distributed)MatMul{XWT,XW,XTW}`` modules.

``DistributedLinear``: ``x`` holds tokens over ``row_group`` and features over
``col_group``; the weight ``(out, in)`` is split into ``(out / Rw, in / C)`` blocks with
``Rw = |model_group| / |col_group|`` (``Rw = 1``, i.e. replicated over ``row_group`` and
marked, when ``model_group is col_group`` as in attention projections); the bias holds
``out / C`` entries, replicated over ``row_group``.  The output is again (row, col)-blocked
so layers chain without gathers.

Forward = all-gather(x over col) -> fetch of the weight rows that make this rank's output block (straight
from the blocks' owners, in the compute dtype) -> one local GEMM (+ bias); any R x C that divides the shapes
is accepted (the reference implements 1x1, 1x2, 2x2 and
4x2 only).  On CUDA the local GEMM runs on the tcgen05 kernel of ``jigsaw_b200.ops``.

Reference parity: jigsaw/modules/linear/_linear.py:55-594 (DistributedLinear), :597-761
(DistributedMatMul*), :776-836 (MatMul*); jigsaw/modules/linear/_functional.py:113-466.
"""

from __future__ import annotations

import math
import warnings
from typing import Any

import torch
import torch.distributed as dist

from ... import init, parallel
from ..._core.autocast import cast_to_autocast_dtype
from ..._core.collectives import all_gather_cat
from ..._core.config import check_config
from ..._core.placement import check_divisible, gather_dim
from ..._core.shard_repr import shard_repr
from ._config import LinearConfig, default_grid
from ._functional import block_matmul, fetch_region


def _local_linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
    if x.is_cuda:
        from ...ops import linear_fused

        out = linear_fused.maybe_fused_linear(x, w, b)
        if out is not None:
            return out
    return torch.nn.functional.linear(x, w, b)


class DistributedLinear(torch.nn.Module):
    def __init__(
        self,
        in_dim: int,
        out_dim: int,
        device: torch.device | str,
        model_group: dist.ProcessGroup,
        row_group: dist.ProcessGroup,
        col_group: dist.ProcessGroup,
        bias: bool = True,
        config: LinearConfig | None = None,
        dtype: torch.dtype = torch.float32,
        *,
        local_rank: int | None = None,
    ) -> None:
        super().__init__()
        if local_rank is not None:
            warnings.warn("local_rank is deprecated and ignored", DeprecationWarning, stacklevel=2)
        self.in_dim, self.out_dim = in_dim, out_dim
        self.device = torch.device(device)
        self.dtype = dtype
        # a layer whose model group is the column group of a mesh with several rows keeps its
        # weight unsplit over rows, and stays that way when resharded; on a one-row mesh the two
        # groups cannot be told apart and the layer counts as fully model-parallel
        self._model_is_col = model_group is col_group and row_group.size() > 1
        self._bind_groups(model_group, row_group, col_group)
        if config is not None:
            check_config(config, {"model group size": model_group.size(), "linear_layer": True})
        self.config = config or LinearConfig(model_group, linear_layer=True, device=self.device)
        self.global_weight_shape = (out_dim, in_dim)
        self.global_bias_shape = (out_dim,) if bias else None
        self.weight = torch.nn.Parameter(
            torch.empty(out_dim // self.row_split, in_dim // self.col_split, device=self.device, dtype=dtype)
        )
        self.bias = (
            torch.nn.Parameter(torch.empty(out_dim // self.col_split, device=self.device, dtype=dtype)) if bias else None
        )
        self.reset_parameters()
        self._mark()

    def _bind_groups(self, model_group: dist.ProcessGroup, row_group: dist.ProcessGroup, col_group: dist.ProcessGroup) -> None:
        """Check that the groups fit this layer, then adopt them (nothing changes when a check fails)."""
        C = col_group.size()
        if model_group.size() % C:
            raise ValueError("model group size must be a multiple of the column group size")
        row_split = model_group.size() // C            # weight row blocks
        if row_split > 1 and row_split != row_group.size():
            raise NotImplementedError(
                f"weight rows are split {row_split}-way but row_group has {row_group.size()} ranks; "
                "model_group must span row_group x col_group or equal col_group"
            )
        check_divisible(self.in_dim, C, "in_dim")
        check_divisible(self.out_dim, row_split, "out_dim")
        if self.out_dim % C:
            raise ValueError(f"out_dim={self.out_dim} must be divisible by the column group size {C}, which shards the bias and the output columns")
        self.model_group, self.row_group, self.col_group = model_group, row_group, col_group
        self.col_split, self.row_split = C, row_split
        self.weight_replicated_over_rows = row_split == 1

    def _mark(self) -> None:
        """Bias is always replicated over ``row_group``; the weight too when its rows are not split."""
        targets = []
        if self.bias is not None:
            targets.append(self.bias)
        if self.weight_replicated_over_rows:
            targets.append(self.weight)
        for p in targets:
            if not parallel.replica_groups(p):
                parallel.mark_replicated(p, [self.row_group])
        if self.row_group.size() > 1:
            with torch.no_grad():
                for p in targets:
                    dist.broadcast(p.data, group_src=0, group=self.row_group)

    def reset_parameters(self) -> None:
        """Same distributions as ``torch.nn.Linear`` (fans from the global shape)."""
        init.kaiming_uniform_(self.weight, a=math.sqrt(5), global_shape=self.global_weight_shape)
        if self.bias is not None:
            bound = 1.0 / math.sqrt(self.in_dim) if self.in_dim > 0 else 0.0
            init.uniform_(self.bias, -bound, bound)

    # ------------------------------------------------------------------ forward
    def _out_block_weight(self, w: torch.Tensor) -> torch.Tensor:
        """The ``(out / C, in)`` rows of the global weight that make this rank's output block, fetched block by
        block from their owners (in the compute dtype): ``R / C`` row blocks times ``C`` column blocks, i.e.
        ``out * in / C`` elements in flight, never the whole matrix."""
        (w,) = cast_to_autocast_dtype(w)
        C, n = self.col_split, self.out_dim // self.col_split
        k = w.shape[1]
        if self.row_split > 1:
            # the weight is cut R x C over the model group (rank i * C + j holds block (i, j))
            return fetch_region(w, self.model_group, self.row_split, C, lambda p: ((p % C) * n, (p % C + 1) * n, 0, k * C),
                                self.config.comm)
        # replicated over rows: cut 1 x C over the column group
        return fetch_region(w, self.col_group, 1, C, lambda p: (p * n, (p + 1) * n, 0, k * C), self.config.comm)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = parallel.sync_grad(self.weight, self.bias)
        w_j = self._out_block_weight(w)                                     # (N/C, K)
        if x.is_cuda and self.col_split > 1:
            from ...ops import linear_fused

            # all-gather of x fused into the GEMM: the kernel reads the peers' blocks itself
            out = linear_fused.maybe_fused_gather_linear(x, w_j, b, self.col_group)
            if out is not None:
                return out
        x_full = all_gather_cat(x, self.col_group, -1)                     # (.., M/R, K)
        return _local_linear(x_full, w_j, b)

    # ------------------------------------------------------------------ conversion
    @classmethod
    def convert_to_jigsaw(
        cls, model: torch.nn.Linear, process_mesh_dict: dict, device: torch.device | str, row_kw: str = "row",
        col_kw: str = "col", model_kw: str = "model", comm: str = "auto", **kwargs: Any,
    ) -> "DistributedLinear":
        mg = process_mesh_dict[model_kw]
        layer = cls(
            model.in_features, model.out_features, device, mg, process_mesh_dict[row_kw], process_mesh_dict[col_kw],
            bias=model.bias is not None, dtype=model.weight.dtype,
            config=LinearConfig(mg, linear_layer=True, device=device, comm=comm),
        )
        layer._load_global(model.weight.data, None if model.bias is None else model.bias.data)
        return layer

    def _load_global(self, weight: torch.Tensor, bias: torch.Tensor | None) -> None:
        i = self.row_group.rank() if self.row_split > 1 else 0
        j = self.col_group.rank()
        rb, cb = self.out_dim // self.row_split, self.in_dim // self.col_split
        with torch.no_grad():
            self.weight.data = weight[i * rb : (i + 1) * rb, j * cb : (j + 1) * cb].clone().to(self.device).contiguous()
            if bias is not None and self.bias is not None:
                nb = self.out_dim // self.col_split
                self.bias.data = bias[j * nb : (j + 1) * nb].clone().to(self.device)

    def merge_weights(
        self, from_process_mesh: dict, row_kw: str = "row", col_kw: str = "col", model_kw: str = "model"
    ) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Global weight and bias from the shards (collective over the row and column groups)."""
        col = from_process_mesh[col_kw]
        with torch.no_grad():
            w = gather_dim(self.weight.detach(), col, 1)
            if self.row_split > 1:
                w = gather_dim(w, from_process_mesh[row_kw], 0)
            b = None if self.bias is None else gather_dim(self.bias.detach(), col, 0)
        return w, b

    def convert_to_torch(self, process_mesh_dict: dict, row_kw: str = "row", col_kw: str = "col", model_kw: str = "model") -> torch.nn.Linear:
        w, b = self.merge_weights(process_mesh_dict, row_kw, col_kw, model_kw)
        layer = torch.nn.Linear(self.in_dim, self.out_dim, bias=b is not None, device=self.device, dtype=w.dtype)
        layer.weight.data = w
        if b is not None:
            layer.bias.data = b
        return layer

    def reshard_parameters(
        self, from_process_mesh: dict, to_process_mesh: dict, pm_row_key: str = "row", pm_col_key: str = "col",
        pm_model_key: str = "model",
    ) -> None:
        """Move the layer to another mesh (collective over both).  The target layout follows the meshes when they
        describe this layer, i.e. when ``from_process_mesh[pm_model_key]`` is the layer's model group: a
        target whose model group is its column group (on a mesh with several rows) gives the column-only layout
        (weight replicated over the rows and marked so), any other target the row x column layout.  When the
        source mesh names another model group (a generic loop that hands every layer the whole mesh, although
        this layer is the column-only projection of an attention block) the layer keeps its kind of layout."""
        def same(a: dist.ProcessGroup, b: dist.ProcessGroup) -> bool:
            return a is b or dist.get_process_group_ranks(a) == dist.get_process_group_ranks(b)

        to_row, to_col = to_process_mesh[pm_row_key], to_process_mesh[pm_col_key]
        from_model = from_process_mesh.get(pm_model_key) if hasattr(from_process_mesh, "get") else None
        if from_model is not None and same(from_model, self.model_group) and pm_model_key in to_process_mesh:
            col_only = same(to_process_mesh[pm_model_key], to_col) and to_row.size() > 1
        else:
            col_only = self._model_is_col
        new_model = to_col if col_only else to_process_mesh[pm_model_key]
        if (self.model_group is new_model and self.row_group is to_process_mesh[pm_row_key]
                and self.col_group is to_process_mesh[pm_col_key]):
            return                                  # already there (a parent layer moved this one with itself)
        w, b = self.merge_weights(from_process_mesh, pm_row_key, pm_col_key, pm_model_key)
        self._bind_groups(new_model, to_process_mesh[pm_row_key], to_process_mesh[pm_col_key])
        self._model_is_col = col_only
        self.config = LinearConfig(new_model, linear_layer=True, device=self.device, comm=self.config.comm)
        self.weight = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=w.dtype))
        if self.bias is not None:
            self.bias = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=w.dtype))
        self._load_global(w, b)
        self._mark()

    def shard_spec(self) -> dict[str, tuple[tuple[int, dist.ProcessGroup], ...]]:
        """Which dimension of which parameter is cut over which group (sharded checkpoints)."""
        w = [(1, self.col_group)]
        if self.row_split > 1:
            w.append((0, self.row_group))
        return {"weight": tuple(w), "bias": ((0, self.col_group),)}

    def get_parameter_count(self) -> int:
        return self.in_dim * self.out_dim + (self.out_dim if self.bias is not None else 0)

    def extra_repr(self) -> str:
        return (
            f"in_features={self.in_dim}, out_features={self.out_dim}, bias={self.bias is not None}, "
            + shard_repr(row=self.row_split, col=self.col_group)
        )


class _DistributedMatMul(torch.nn.Module):
    _kind = "xwt"

    def __init__(self, device: torch.device | str, model_group: dist.ProcessGroup | None, config: LinearConfig | None = None,
                 *, local_rank: int | None = None) -> None:
        super().__init__()
        if local_rank is not None:
            warnings.warn("local_rank is deprecated and ignored", DeprecationWarning, stacklevel=2)
        self.device = torch.device(device)
        self.model_group = model_group                      # None: a single process, no process group needed
        size = 1 if model_group is None else model_group.size()
        self.grid = default_grid(size)
        if config is not None:
            check_config(config, {"model group size": size, "linear_layer": False})
        self.config = config or LinearConfig(model_group, linear_layer=False, device=self.device)

    def forward(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return block_matmul(self._kind, x, w, self.model_group, *self.grid, comm=self.config.comm)

    def get_parameter_count(self) -> int:
        return 0

    def extra_repr(self) -> str:
        return shard_repr(model=self.model_group)


class DistributedMatMulXWT(_DistributedMatMul):
    """``Y = X W^T`` on 2-D block-distributed operands."""

    _kind = "xwt"


class DistributedMatMulXW(_DistributedMatMul):
    """``Y = X W`` on 2-D block-distributed operands."""

    _kind = "xw"


class DistributedMatMulXTW(_DistributedMatMul):
    """``Y = X^T W`` on 2-D block-distributed operands."""

    _kind = "xtw"


class _MatMul(torch.nn.Module):
    def get_parameter_count(self) -> int:
        return 0


class MatMulXWT(_MatMul):
    """Serial ``X W^T`` (convertible to :class:`DistributedMatMulXWT`)."""

    def forward(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        x, w = cast_to_autocast_dtype(x, w)
        return torch.matmul(x, w.transpose(-1, -2))


class MatMulXW(_MatMul):
    """Serial ``X W``."""

    def forward(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        x, w = cast_to_autocast_dtype(x, w)
        return torch.matmul(x, w)


class MatMulXTW(_MatMul):
    """Serial ``X^T W``."""

    def forward(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        x, w = cast_to_autocast_dtype(x, w)
        return torch.matmul(x.transpose(-1, -2), w)


def _convert_matmul(dist_cls: type) -> Any:
    def convert(cls: type, model: torch.nn.Module, process_mesh_dict: dict, device: torch.device | str,
                row_kw: str = "row", col_kw: str = "col", model_kw: str = "model", comm: str = "auto", **kw: Any) -> Any:
        mg = process_mesh_dict[model_kw]
        return dist_cls(device, mg, LinearConfig(mg, linear_layer=False, device=device, comm=comm))

    return classmethod(convert)


for _serial, _dist in ((MatMulXWT, DistributedMatMulXWT), (MatMulXW, DistributedMatMulXW), (MatMulXTW, DistributedMatMulXTW)):
    _dist.convert_to_jigsaw = _convert_matmul(_dist)
    _dist.convert_to_torch = (lambda s: (lambda self, *a, **k: s()))(_serial)
