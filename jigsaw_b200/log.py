"""Rank-aware logging for one-process-per-GPU jobs.

Every record is stamped with ``rank/world``, the local rank and the seconds since import.
Plain calls (:func:`info`, ...) print on one *print rank* only; ``*_all`` and :func:`at`
address other ranks.  Output is human-readable (optionally coloured) or JSON lines, on
stderr and optionally in per-rank files ``rank_<NNNN>.log``.

Environment (explicit arguments of :func:`configure_logging` win):
``JIGSAW_LOG_LEVEL`` (default ``INFO``), ``JIGSAW_LOG_RANK`` (print rank, default 0),
``JIGSAW_LOG_DIR`` (per-rank files), ``JIGSAW_LOG_FORMAT=json``.

Fail-together helpers live here too: :func:`assert_all_agree` (collective config check),
:func:`die`, and an excepthook that logs the traceback with the rank and destroys the
process group so a crashing rank fails the job instead of dead-locking its peers.

Reference parity: jigsaw/log.py:48-68 (API), :122-184 (filter / formatters), :190-312
(configure), :406-457 (rank scoping), :460-561 (once / ranks / agree), :564-663 (timed,
die, excepthook).
"""

from __future__ import annotations

import faulthandler
import json
import logging
import os
import platform
import signal
import sys
import time
import warnings as _warnings
from collections.abc import Iterable, Iterator
from contextlib import contextmanager
from pathlib import Path
from typing import Any, NoReturn

import torch
import torch.distributed as dist

__all__ = [
    "configure_logging",
    "get_logger",
    "set_print_rank",
    "at",
    "only_rank",
    "debug",
    "info",
    "warning",
    "error",
    "exception",
    "debug_all",
    "info_all",
    "warning_all",
    "error_all",
    "log_once",
    "log_ranks",
    "assert_all_agree",
    "timed",
    "die",
]

LOGGER_NAME = "jigsaw"
_T0 = time.monotonic()
_state: dict[str, Any] = {"configured": False, "print_rank": 0, "scope": None}
_once_keys: set[tuple[str, int, str]] = set()
_logger = logging.getLogger(LOGGER_NAME)


def _env_int(*names: str, default: int) -> int:
    for n in names:
        v = os.environ.get(n)
        if v is not None and v.lstrip("-").isdigit():
            return int(v)
    return default


def _rank_world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return _env_int("RANK", "SLURM_PROCID", default=0), _env_int("WORLD_SIZE", "SLURM_NTASKS", default=1)


def _local_rank() -> int:
    return _env_int("LOCAL_RANK", "SLURM_LOCALID", default=0)


def _targets(spec: Any) -> set[int] | None:
    """``None`` = every rank; otherwise the set of addressed ranks."""
    if spec is None:
        return {_state["print_rank"]}
    if isinstance(spec, str):
        if spec.lower() == "all":
            return None
        raise ValueError(f"rank spec must be an int, ints or 'all', got {spec!r}")
    if isinstance(spec, int):
        return {spec}
    if isinstance(spec, Iterable):
        return {int(r) for r in spec}
    raise ValueError(f"rank spec must be an int, ints or 'all', got {spec!r}")


class _Stamp(logging.Filter):
    """Adds rank fields to a record and drops it on ranks it is not addressed to."""

    def filter(self, record: logging.LogRecord) -> bool:
        rank, world = _rank_world()
        record.rank, record.world, record.local_rank = rank, world, _local_rank()
        record.elapsed = time.monotonic() - _T0
        spec = getattr(record, "target_ranks", None)
        if spec is None and _state["scope"] is not None:
            spec = _state["scope"]
        wanted = _targets(spec)
        return wanted is None or rank in wanted


_COLOURS = {"DEBUG": "\033[2m", "INFO": "", "WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[1;31m"}


class _Human(logging.Formatter):
    def __init__(self, colour: bool) -> None:
        super().__init__()
        self.colour = colour

    def format(self, record: logging.LogRecord) -> str:
        head = "[%8.3fs r%d/%d %s] " % (
            getattr(record, "elapsed", 0.0),
            getattr(record, "rank", 0),
            getattr(record, "world", 1),
            record.levelname[0],
        )
        text = head + record.getMessage()
        if record.exc_info:
            text += "\n" + self.formatException(record.exc_info)
        if self.colour and _COLOURS.get(record.levelname):
            text = _COLOURS[record.levelname] + text + "\033[0m"
        return text


class _Json(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        doc = {
            "t": round(getattr(record, "elapsed", 0.0), 6),
            "rank": getattr(record, "rank", 0),
            "world": getattr(record, "world", 1),
            "local_rank": getattr(record, "local_rank", 0),
            "level": record.levelname,
            "logger": record.name,
            "msg": record.getMessage(),
        }
        if record.exc_info:
            doc["exc"] = self.formatException(record.exc_info)
        return json.dumps(doc)


def configure_logging(
    level: str | int | None = None,
    *,
    rank: int | None = None,
    log_dir: str | os.PathLike[str] | None = None,
    as_json: bool | None = None,
    colour: bool | None = None,
    capture_warnings: bool = True,
    install_excepthook: bool = True,
    enable_faulthandler: bool = True,
    force: bool = False,
) -> logging.Logger:
    """Install the handlers of the ``jigsaw`` logger (idempotent unless ``force``)."""
    if _state["configured"] and not force:
        return _logger
    if level is None:
        level = os.environ.get("JIGSAW_LOG_LEVEL", "INFO")
    if rank is None:
        rank = _env_int("JIGSAW_LOG_RANK", default=0)
    _state["print_rank"] = rank
    if log_dir is None:
        log_dir = os.environ.get("JIGSAW_LOG_DIR") or None
    if as_json is None:
        as_json = os.environ.get("JIGSAW_LOG_FORMAT", "").lower() == "json"
    if colour is None:
        colour = sys.stderr.isatty() and os.environ.get("NO_COLOR") is None

    for h in list(_logger.handlers):
        _logger.removeHandler(h)
        h.close()
    stamp = _Stamp()
    console = logging.StreamHandler(sys.stderr)
    console.setFormatter(_Json() if as_json else _Human(colour))
    console.addFilter(stamp)
    _logger.addHandler(console)
    if log_dir is not None:
        path = Path(log_dir)
        path.mkdir(parents=True, exist_ok=True)
        me, _ = _rank_world()
        fileh = logging.FileHandler(path / f"rank_{me:04d}.log")
        fileh.setFormatter(_Json() if as_json else _Human(False))

        class _AllRanks(_Stamp):
            # the per-rank file keeps every record of its own rank
            def filter(self, record: logging.LogRecord) -> bool:
                super().filter(record)
                return True

        fileh.addFilter(_AllRanks())
        _logger.addHandler(fileh)
    _logger.setLevel(level if isinstance(level, int) else str(level).upper())
    _logger.propagate = False
    if capture_warnings:
        logging.captureWarnings(True)
        wl = logging.getLogger("py.warnings")
        for h in _logger.handlers:
            if h not in wl.handlers:
                wl.addHandler(h)
    if install_excepthook:
        _install_excepthook()
    if enable_faulthandler:
        try:
            faulthandler.enable()
            if hasattr(signal, "SIGUSR1"):
                faulthandler.register(signal.SIGUSR1, all_threads=True, chain=True)
        except (RuntimeError, ValueError, OSError, AttributeError):
            pass
    _state["configured"] = True
    return _logger


def get_logger(name: str | None = None) -> logging.Logger:
    """Return the ``jigsaw`` logger or a child ``jigsaw.<name>`` that shares its handlers."""
    if name is None or name == LOGGER_NAME:
        return _logger
    if name.startswith(LOGGER_NAME + "."):
        return logging.getLogger(name)
    return _logger.getChild(name)


class _Addressed:
    """Logging front-end whose records are addressed to a fixed rank set."""

    def __init__(self, ranks: Any) -> None:
        self.ranks = ranks

    def _emit(self, level: int, msg: str, args: tuple, exc_info: Any = None) -> None:
        if not _state["configured"]:
            configure_logging()
        if _logger.isEnabledFor(level):
            extra = {} if self.ranks is None else {"target_ranks": self.ranks}
            _logger.log(level, msg, *args, exc_info=exc_info, extra=extra, stacklevel=3)

    def debug(self, msg: str, *args: object) -> None:
        self._emit(logging.DEBUG, msg, args)

    def info(self, msg: str, *args: object) -> None:
        self._emit(logging.INFO, msg, args)

    def warning(self, msg: str, *args: object) -> None:
        self._emit(logging.WARNING, msg, args)

    def error(self, msg: str, *args: object) -> None:
        self._emit(logging.ERROR, msg, args)

    def exception(self, msg: str, *args: object) -> None:
        self._emit(logging.ERROR, msg, args, exc_info=True)


_default = _Addressed(None)
_everyone = _Addressed("all")

debug, info, warning, error, exception = (
    _default.debug,
    _default.info,
    _default.warning,
    _default.error,
    _default.exception,
)
debug_all, info_all, warning_all, error_all = _everyone.debug, _everyone.info, _everyone.warning, _everyone.error


def at(ranks: Any) -> _Addressed:
    """Logger addressed to ``ranks`` (an int, an iterable of ints or ``"all"``)."""
    _targets(ranks)  # validate now
    return _Addressed(ranks)


def set_print_rank(rank: int) -> None:
    """Change the rank that plain calls print on."""
    _state["print_rank"] = int(rank)


@contextmanager
def only_rank(ranks: Any) -> Iterator[None]:
    """Inside the block, plain calls are addressed to ``ranks`` instead of the print rank."""
    _targets(ranks)
    previous = _state["scope"]
    _state["scope"] = ranks
    try:
        yield
    finally:
        _state["scope"] = previous


def log_once(msg: str, *args: object, level: int = logging.INFO) -> None:
    """Log only the first time this call site (file, line, message) is reached."""
    frame = sys._getframe(1)
    key = (frame.f_code.co_filename, frame.f_lineno, msg)
    if key in _once_keys:
        return
    _once_keys.add(key)
    _default._emit(level, msg, args)


def log_ranks(msg: str, *args: object, level: int = logging.DEBUG, group: dist.ProcessGroup | None = None) -> None:
    """Collective: gather one line per rank and print them in rank order from group rank 0."""
    if not _logger.isEnabledFor(level):
        return
    rank, world = _rank_world()
    line = (msg % args) if args else msg
    if not (dist.is_available() and dist.is_initialized()) or world == 1:
        _default._emit(level, "%s", (line,))
        return
    lines: list[Any] = [None] * dist.get_world_size(group)
    dist.all_gather_object(lines, f"[{rank}] {line}", group=group)
    if dist.get_rank(group) == 0:
        _everyone._emit(level, "rank dump:\n%s", ("\n".join(map(str, lines)),))


def assert_all_agree(name: str, value: object, *, group: dist.ProcessGroup | None = None, fatal: bool = True) -> bool:
    """Collective check that ``value`` (picklable, ``==``-comparable) is the same on every rank."""
    if not (dist.is_available() and dist.is_initialized()):
        return True
    world = dist.get_world_size(group)
    if world == 1:
        return True
    seen: list[Any] = [None] * world
    dist.all_gather_object(seen, value, group=group)
    if all(v == seen[0] for v in seen):
        return True
    if dist.get_rank(group) == 0:
        detail = ", ".join(f"r{i}={v!r}" for i, v in enumerate(seen))
        _everyone._emit(logging.ERROR, "ranks disagree on %s: %s", (name, detail))
    if fatal:
        die("ranks disagree on %r", name)
    return False


@contextmanager
def timed(
    label: str,
    *,
    level: int = logging.INFO,
    barrier: bool = False,
    cuda_sync: bool = False,
    group: dist.ProcessGroup | None = None,
) -> Iterator[None]:
    """Wall-clock a block and log ``"<label> took X s"`` from the print rank."""
    live = dist.is_available() and dist.is_initialized()
    if barrier and live:
        dist.barrier(group=group)
    t0 = time.perf_counter()
    try:
        yield
    finally:
        if cuda_sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        if barrier and live:
            dist.barrier(group=group)
        _default._emit(level, "%s took %.3f s", (label, time.perf_counter() - t0))


def _teardown() -> None:
    if dist.is_available() and dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001 - shutdown path
            pass


def die(msg: str, *args: object, code: int = 1) -> NoReturn:
    """Log a fatal message on every rank, flush, destroy the process group and ``os._exit``."""
    _everyone._emit(logging.CRITICAL, msg, args)
    for h in _logger.handlers:
        h.flush()
    _teardown()
    os._exit(code)


def _install_excepthook() -> None:
    previous = sys.excepthook
    if getattr(previous, "_jigsaw_hook", False):
        return

    def hook(exc_type, exc, tb):  # type: ignore[no-untyped-def]
        if issubclass(exc_type, KeyboardInterrupt):
            previous(exc_type, exc, tb)
            return
        rank, world = _rank_world()
        _logger.critical(
            "uncaught exception on rank %d/%d (%s)",
            rank,
            world,
            platform.node(),
            exc_info=(exc_type, exc, tb),
            extra={"target_ranks": "all"},
        )
        for h in _logger.handlers:
            h.flush()
        _teardown()

    hook._jigsaw_hook = True  # type: ignore[attr-defined]
    sys.excepthook = hook


# keep ``warnings`` importable under its usual name for callers of this module
warnings = _warnings
