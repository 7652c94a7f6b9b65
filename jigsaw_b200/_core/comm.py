"""Communication primitives: backend checks, transport selection, sparse exchanges.

One primitive carries every neighbour pattern of the library: :func:`sparse_exchange`
moves a different tensor to / from each peer of a group (absent peers cost nothing).
The halo gather, the ring hop and the roll swap are all particular send / receive
tables for it.  Three interchangeable ``torch.distributed`` transports implement it
(``CommOp``); on CUDA the fused sm_100a kernels bypass it entirely and store into peer
memory, so this module is the CPU path, the parity oracle and the measured baseline.

Reference parity: jigsaw/_core/comm.py:16-46 (backend check), :80-137 (CommOp and its
resolution), :239-417 (1-D neighbour exchanges), :430-505 (async all-to-all, broadcast,
max-reduce).
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from enum import Enum
from functools import lru_cache

import torch
import torch.distributed as dist

_SUPPORTED = {"nccl": "cuda", "gloo": "cpu"}


def check_backend(group: dist.ProcessGroup | None = None) -> set[str]:
    """Return the backend names of ``group``; raise ``RuntimeError`` for unsupported ones.

    ``"nccl"`` and ``"gloo"`` are supported, also mixed as ``"cpu:gloo,cuda:nccl"``.
    Any other backend would take the NCCL code paths and hang, so it is refused early.
    """
    backend = str(dist.get_backend(group))
    names = {part.split(":")[-1] for part in backend.split(",")}
    bad = names - set(_SUPPORTED)
    if bad:
        raise RuntimeError(
            f"unsupported process-group backend {backend!r}; supported: {sorted(_SUPPORTED)}"
        )
    return names


def get_device_of_process_group(group: dist.ProcessGroup | None = None) -> torch.device:
    """Device that tensors must live on for collectives over ``group``."""
    if "nccl" in check_backend(group):
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


class CommOp(str, Enum):
    """Transport of the neighbour exchanges of a distributed layer.

    ``AUTO`` picks ``ALL_TO_ALL`` on CUDA (one fused NCCL launch, zero-length entries for
    idle peers) and ``BATCH_ISEND_IRECV`` on CPU (gloo's all-to-all rejects empty
    entries).  ``ISEND`` issues separate ``isend`` / ``irecv`` and is CPU-only: separate
    NCCL sends around a ring can deadlock.  Strings are accepted in any case.
    """

    AUTO = "auto"
    ALL_TO_ALL = "all_to_all"
    ISEND = "isend"
    BATCH_ISEND_IRECV = "batch_isend_irecv"

    def __str__(self) -> str:  # StrEnum behaviour
        return self.value


def resolve_comm_op(comm: CommOp | str, device: torch.device | str) -> CommOp:
    """Turn ``comm`` (enum or case-insensitive string) into a concrete transport for ``device``."""
    device = torch.device(device)
    if device.type not in ("cuda", "cpu"):
        raise ValueError(f"Unsupported device {device.type}")
    if not isinstance(comm, CommOp):
        key = str(comm).lower()
        values = [m.value for m in CommOp]
        if key not in values:
            raise ValueError(f"comm must be one of {values}, got {comm!r}")
        comm = CommOp(key)
    if comm is CommOp.AUTO:
        return CommOp.ALL_TO_ALL if device.type == "cuda" else CommOp.BATCH_ISEND_IRECV
    if comm is CommOp.ALL_TO_ALL and device.type != "cuda":
        raise ValueError(
            f"comm='all_to_all' needs CUDA (NCCL), got device {device.type!r}; "
            "use 'isend' or 'batch_isend_irecv'"
        )
    if comm is CommOp.ISEND and device.type == "cuda":
        return CommOp.BATCH_ISEND_IRECV
    return comm


@lru_cache(maxsize=None)
def _empty(dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """Cached zero-length placeholder (idle peers of an all-to-all)."""
    return torch.empty(0, dtype=dtype, device=device)


class ExchangeWork:
    """Handle of an asynchronous :func:`sparse_exchange`; ``wait()`` completes it."""

    def __init__(self, works: Sequence[dist.Work | None]):
        self._works = [w for w in works if w is not None]

    def wait(self) -> None:
        for w in self._works:
            w.wait()
        self._works = []


def sparse_exchange(
    sends: Mapping[int, torch.Tensor],
    recvs: Mapping[int, torch.Tensor],
    group: dist.ProcessGroup,
    comm: CommOp = CommOp.BATCH_ISEND_IRECV,
    async_op: bool = False,
) -> ExchangeWork | None:
    """Send ``sends[p]`` to group rank ``p`` and receive into ``recvs[p]`` from group rank ``p``.

    Every rank of ``group`` must call it (with possibly empty tables).  Tensors must be
    contiguous.  Entries addressed to the calling rank itself are copied locally.

    Returns ``None`` when complete, or an :class:`ExchangeWork` when ``async_op``.
    """
    me = group.rank()
    size = group.size()
    if me in sends and me in recvs:
        recvs[me].copy_(sends[me])
    sends = {p: t for p, t in sends.items() if p != me and t.numel() > 0}
    recvs = {p: t for p, t in recvs.items() if p != me and t.numel() > 0}
    works: list[dist.Work | None] = []
    if comm is CommOp.ALL_TO_ALL:
        some = next(iter(sends.values()), None)
        if some is None:
            some = next(iter(recvs.values()), None)
        if some is None:
            # keep the collective matched on every rank: an all-empty all-to-all
            dev = get_device_of_process_group(group)
            dtype = torch.float32
        else:
            dev, dtype = some.device, some.dtype
        out_list = [recvs.get(p, _empty(dtype, dev)).view(-1) for p in range(size)]
        in_list = [sends.get(p, _empty(dtype, dev)).reshape(-1) for p in range(size)]
        works.append(dist.all_to_all(out_list, in_list, group=group, async_op=async_op))
    elif comm is CommOp.ISEND:
        # receives first so that a blocking wait order can never deadlock
        for p in sorted(recvs):
            works.append(dist.irecv(recvs[p], group=group, group_src=p))
        for p in sorted(sends):
            works.append(dist.isend(sends[p], group=group, group_dst=p))
        if not async_op:
            for w in works:
                w.wait()
            works = []
    else:
        ops = [dist.P2POp(dist.irecv, recvs[p], group=group, group_peer=p) for p in sorted(recvs)]
        ops += [dist.P2POp(dist.isend, sends[p], group=group, group_peer=p) for p in sorted(sends)]
        if ops:
            works = list(dist.batch_isend_irecv(ops))
        if not async_op:
            for w in works:
                w.wait()
            works = []
    if async_op:
        return ExchangeWork(works)
    for w in works:
        if w is not None:
            w.wait()
    return None


def ring_shift(
    data: torch.Tensor,
    buffer: torch.Tensor | None,
    direction: int,
    group: dist.ProcessGroup,
    comm: CommOp = CommOp.BATCH_ISEND_IRECV,
    async_op: bool = False,
) -> tuple[torch.Tensor, ExchangeWork | None]:
    """Cyclic 1-D neighbour exchange: send ``data`` to rank ``r + direction`` and receive
    the block of rank ``r - direction`` into ``buffer`` (allocated when ``None``).

    Returns ``(buffer, work)``; ``work`` is ``None`` unless ``async_op``.
    """
    size, me = group.size(), group.rank()
    if buffer is None:
        buffer = torch.empty_like(data)
    if size == 1:
        buffer.copy_(data)
        return buffer, None
    dst = (me + direction) % size
    src = (me - direction) % size
    work = sparse_exchange({dst: data.contiguous()}, {src: buffer}, group, comm, async_op)
    return buffer, work




def all_reduce_max(value: float | int, group: dist.ProcessGroup | None = None) -> float:
    """MAX-reduce a Python scalar so that every rank takes the same decision."""
    dev = get_device_of_process_group(group)
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
