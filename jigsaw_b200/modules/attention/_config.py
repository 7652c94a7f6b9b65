"""Policies of ring attention: what travels, what is saved, how dK/dV return, which core.

All enums accept their member, or its name as a string in any case; ``AttnBackend`` also
accepts its value (``"sdpa"``).  ``RingAttentionConfig`` validates the combination once
at construction.

Reference parity: jigsaw/modules/attention/_config.py:17-85 (enums), :91-133 (coercion),
:339-524 (RingAttentionConfig).
"""

from __future__ import annotations

from enum import Enum
from typing import Any

import torch

from ..._core.comm import CommOp, resolve_comm_op


class SendForward(Enum):
    """What circulates in the forward pass: the layer input (K/V recomputed per hop) or K/V."""

    X = 0
    KV = 1


class SaveBackward(Enum):
    """What is kept for the backward pass."""

    X = 0
    KV = 1


class SaveScope(Enum):
    """``LOCAL``: keep only the own chunk and fetch the others again in backward (memory
    constant in the ring size).  ``GLOBAL``: keep every chunk that arrived."""

    LOCAL = 0
    GLOBAL = 1


class Offload(Enum):
    """Where saved chunks live between forward and backward."""

    DISABLED = 0
    CPU = 1


class SendBackward(Enum):
    """``SEND_DKV``: each step's dK/dV goes straight to the chunk owner.  ``GATHER_DKV``:
    accumulate all chunks' dK/dV locally and reduce once at the end."""

    SEND_DKV = 0
    GATHER_DKV = 1


class SendOp(Enum):
    """Order in which a rank visits the chunks (see ``chunk_owner``): neighbour ring,
    owner broadcast, or the two-level variants with intra groups of ``intra_size``."""

    RING = 0
    BROADCAST = 1
    HYBRID = 2
    HYBRID_BROADCAST = 3


class AttnBackend(str, Enum):
    """Attention core: ``SDPA`` (fused flash kernels on CUDA, math on CPU), ``MATH`` (unfused
    reference, any device / dtype), ``TE`` (TransformerEngine; resolved to ``SDPA`` when absent)."""

    TE = "te"
    SDPA = "sdpa"
    MATH = "math"


def coerce_enum(enum_cls: type[Enum], value: Any, arg: str) -> Any:
    """Return ``value`` as a member of ``enum_cls`` or raise ``ValueError``."""
    if isinstance(value, enum_cls):
        return value
    if isinstance(value, str):
        for m in enum_cls:
            if m.name.lower() == value.lower() or (isinstance(m.value, str) and m.value == value.lower()):
                return m
    raise ValueError(f"{arg} must be one of {[m.name for m in enum_cls]}, got {value!r}")


try:  # TransformerEngine is optional and absent from most installations
    import transformer_engine  # noqa: F401

    JIGSAW_TE_AVAILABLE = True
except Exception:  # noqa: BLE001
    JIGSAW_TE_AVAILABLE = False


def resolve_backend(backend: AttnBackend) -> AttnBackend:
    """``TE`` stands for TransformerEngine's fused attention.  It is not used by this library: the request is
    answered with the SDPA backend (the library's own flash kernels on a B200) and a warning, so that a configuration
    written for an installation with TransformerEngine keeps running and says what it runs on."""
    if backend is AttnBackend.TE and not JIGSAW_TE_AVAILABLE:
        import warnings

        warnings.warn("attn_backend='te' needs transformer_engine, which is not installed: falling back to 'sdpa'",
                      UserWarning, stacklevel=3)
        return AttnBackend.SDPA
    return backend


class RingAttentionConfig:
    """Validated bundle of ring-attention policies."""

    def __init__(
        self,
        device: torch.device | str = "cuda",
        send_in_forward: SendForward | str = SendForward.X,
        send_op: SendOp | str = SendOp.RING,
        save_for_backward: SaveBackward | str = SaveBackward.KV,
        save_scope: SaveScope | str = SaveScope.GLOBAL,
        send_backward: SendBackward | str = SendBackward.SEND_DKV,
        offload: Offload | str = Offload.DISABLED,
        intra_size: int = 4,
        attn_backend: AttnBackend | str = AttnBackend.SDPA,
        overlap_comm: bool = False,
        comm: CommOp | str = "auto",
        outer_comm: CommOp | str | None = None,
    ) -> None:
        self.device = torch.device(device)
        self.send_in_forward = coerce_enum(SendForward, send_in_forward, "send_in_forward")
        self.send_op = coerce_enum(SendOp, send_op, "send_op")
        self.save_for_backward = coerce_enum(SaveBackward, save_for_backward, "save_for_backward")
        self.save_scope = coerce_enum(SaveScope, save_scope, "save_scope")
        self.send_backward = coerce_enum(SendBackward, send_backward, "send_backward")
        self.offload = coerce_enum(Offload, offload, "offload")
        self.attn_backend = coerce_enum(AttnBackend, attn_backend, "attn_backend")
        self.attn_backend = resolve_backend(self.attn_backend)
        self.intra_size = int(intra_size)
        self.overlap_comm = bool(overlap_comm)
        self.comm = resolve_comm_op(comm, self.device)
        self.outer_comm = self.comm if outer_comm is None else resolve_comm_op(outer_comm, self.device)
        if self.offload is Offload.CPU and self.save_scope is not SaveScope.GLOBAL:
            raise ValueError("offload=CPU keeps arrived chunks on the host, which needs save_scope=GLOBAL")
        if self.offload is Offload.CPU and self.device.type != "cuda":
            raise ValueError("offload=CPU needs a CUDA device")
        if self.intra_size < 1:
            raise ValueError(f"intra_size must be a positive number of ranks per intra group, got {intra_size}")
        self._layer_key: dict = {}
        self._comm_stream: Any = None
        self._offloader: Any = None

    def __repr__(self) -> str:
        """Every policy by name, so that a log line or an error message says how the ring is run."""
        fields = ("send_in_forward", "send_op", "save_for_backward", "save_scope", "send_backward", "offload", "attn_backend")
        policies = ", ".join(f"{name}={getattr(self, name).name}" for name in fields)
        return (f"RingAttentionConfig(device={str(self.device)!r}, {policies}, intra_size={self.intra_size}, "
                f"overlap_comm={self.overlap_comm}, comm={str(self.comm)!r}, outer_comm={str(self.outer_comm)!r})")

    @property
    def comm_stream(self) -> Any:
        """Side stream used when ``overlap_comm`` is active on CUDA."""
        if self._comm_stream is None and self.device.type == "cuda":
            self._comm_stream = torch.cuda.Stream(device=self.device)
        return self._comm_stream

    @property
    def overlap_active(self) -> bool:
        return self.overlap_comm

    @property
    def offloader(self) -> Any:
        if self._offloader is None:
            from ..._core.offload import ActivationOffloader

            self._offloader = ActivationOffloader(self.device)
        return self._offloader

    def wait_offloads(self) -> None:
        if self._offloader is not None:
            self._offloader.wait_offloads()

    @property
    def core_layout(self) -> str:
        """Layout the attention core works in: ``bshd`` for TE, else ``bhsd``."""
        return "bshd" if self.attn_backend is AttnBackend.TE else "bhsd"
