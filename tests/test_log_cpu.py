"""Rank-aware logging: who speaks (print rank, ``at``, ``only_rank``, ``*_all``), once-only records, rank metadata,
launcher variables, logger names, formatters, configuration (idempotence, environment defaults, per-rank files,
warnings capture), the uncaught-exception hook.

Reference behaviours covered: tests/test_log.py:55-202 (targeting, metadata, launcher variables, proxies, disabled
levels, scope restoration), :204-250 (formatters), :292-360 (configuration).
"""

import io
import json
import logging
import sys
import warnings

import pytest

from jigsaw_b200 import log


@pytest.fixture
def captured(monkeypatch):
    """Configure the logger into a string buffer as JSON and restore the global state afterwards."""
    logger = log.get_logger()
    saved = (list(logger.handlers), logger.level, logger.propagate, dict(log._state), sys.excepthook)
    log.configure_logging("DEBUG", rank=0, as_json=True, install_excepthook=False, enable_faulthandler=False,
                          capture_warnings=False, force=True)
    stream = io.StringIO()
    logger.handlers[0].stream = stream
    log._once_keys.clear()

    def lines():
        return [json.loads(row) for row in stream.getvalue().splitlines()]

    yield lines
    for h in list(logger.handlers):
        logger.removeHandler(h)
    for h in saved[0]:
        logger.addHandler(h)
    logger.setLevel(saved[1])
    logger.propagate = saved[2]
    log._state.clear()
    log._state.update(saved[3])
    sys.excepthook = saved[4]


def _as(monkeypatch, rank, world):
    monkeypatch.setattr(log, "_rank_world", lambda: (rank, world))


def test_only_the_print_rank_speaks_by_default(captured, monkeypatch):
    _as(monkeypatch, 0, 4)
    log.info("hello %d", 1)
    _as(monkeypatch, 3, 4)
    log.info("suppressed")
    assert [rec["msg"] for rec in captured()] == ["hello 1"]
    log.set_print_rank(3)
    log.info("now from 3")
    _as(monkeypatch, 0, 4)
    log.info("no longer from 0")
    assert [rec["msg"] for rec in captured()] == ["hello 1", "now from 3"]


def test_at_targets_an_int_a_list_and_all(captured, monkeypatch):
    _as(monkeypatch, 2, 4)
    log.at(2).info("int")
    log.at([1, 2]).warning("list")
    log.at("all").info("all")
    log.at(1).info("not mine")
    log.at([0, 3]).info("not mine either")
    log.info_all("everyone, whatever the print rank")
    assert [rec["msg"] for rec in captured()] == ["int", "list", "all", "everyone, whatever the print rank"]
    with pytest.raises(ValueError):
        log.at("some")


def test_only_rank_scopes_plain_calls_and_restores_on_error(captured, monkeypatch):
    _as(monkeypatch, 1, 4)
    log.info("outside: print rank is 0")
    with log.only_rank(1):
        log.info("inside")
        log.at(0).info("explicit address wins")
    with pytest.raises(RuntimeError):
        with log.only_rank(1):
            raise RuntimeError
    log.info("outside again")
    assert [rec["msg"] for rec in captured()] == ["inside"]
    assert log._state["scope"] is None


def test_log_once_fires_a_single_time_per_call_site(captured, monkeypatch):
    _as(monkeypatch, 0, 1)
    for _ in range(3):
        log.log_once("once")
    log.log_once("once")                    # another call site
    assert [rec["msg"] for rec in captured()].count("once") == 2


def test_records_carry_rank_metadata_and_levels(captured, monkeypatch):
    _as(monkeypatch, 3, 16)
    log.at("all").debug("d")
    log.at("all").error("e")
    try:
        raise ValueError("boom")
    except ValueError:
        log.at("all").exception("caught")
    got = captured()
    assert [(rec["rank"], rec["world"]) for rec in got] == [(3, 16)] * 3
    assert [rec["level"] for rec in got] == ["DEBUG", "ERROR", "ERROR"]
    assert "ValueError: boom" in got[-1]["exc"] and isinstance(got[0]["t"], float)


def test_a_disabled_level_is_dropped_before_formatting(captured, monkeypatch):
    _as(monkeypatch, 0, 1)
    log.get_logger().setLevel(logging.ERROR)

    class Exploding:
        def __str__(self):
            raise AssertionError("formatted a disabled record")

    log.info("%s", Exploding())
    assert captured() == []


def test_rank_and_world_come_from_the_launcher_without_a_process_group(monkeypatch):
    for var in ("RANK", "WORLD_SIZE", "SLURM_PROCID", "SLURM_NTASKS", "LOCAL_RANK", "SLURM_LOCALID"):
        monkeypatch.delenv(var, raising=False)
    assert log._rank_world() == (0, 1) and log._local_rank() == 0
    monkeypatch.setenv("SLURM_PROCID", "3")
    monkeypatch.setenv("SLURM_NTASKS", "8")
    monkeypatch.setenv("SLURM_LOCALID", "2")
    assert log._rank_world() == (3, 8) and log._local_rank() == 2
    monkeypatch.setenv("RANK", "5")              # torchrun wins over Slurm
    monkeypatch.setenv("WORLD_SIZE", "6")
    monkeypatch.setenv("LOCAL_RANK", "1")
    assert log._rank_world() == (5, 6) and log._local_rank() == 1
    monkeypatch.delenv("WORLD_SIZE")
    monkeypatch.delenv("SLURM_NTASKS")
    assert log._rank_world() == (5, 1)


@pytest.mark.parametrize("name, expected", [(None, "jigsaw"), ("jigsaw", "jigsaw"), ("jigsaw.attn", "jigsaw.attn"), ("attn.ring", "jigsaw.attn.ring")])
def test_loggers_live_under_one_namespace(name, expected):
    assert log.get_logger(name).name == expected


def _record(level=logging.INFO, exc_info=None):
    record = logging.LogRecord("jigsaw.sub", level, __file__, 1, "msg %d", (7,), exc_info)
    record.rank, record.world, record.local_rank, record.elapsed = 2, 4, 0, 1.5
    return record


def test_formatters():
    plain = log._Human(colour=False).format(_record())
    assert "\n" not in plain and plain.endswith("msg 7") and "r2/4" in plain and "1.500s" in plain
    coloured = log._Human(colour=True)
    warn = coloured.format(_record(logging.WARNING))
    assert warn.startswith("\033[33m") and warn.endswith("\033[0m")
    assert "\033" not in coloured.format(_record(logging.INFO))
    try:
        raise KeyError("k")
    except KeyError:
        exc_info = sys.exc_info()
    text = log._Human(colour=False).format(_record(exc_info=exc_info))
    assert "Traceback" in text and "KeyError" in text
    doc = json.loads(log._Json().format(_record()))
    assert doc == {"t": 1.5, "rank": 2, "world": 4, "local_rank": 0, "level": "INFO", "logger": "jigsaw.sub", "msg": "msg 7"}
    assert "KeyError" in json.loads(log._Json().format(_record(exc_info=exc_info)))["exc"]


def test_configuration_is_idempotent_reads_the_environment_and_writes_rank_files(captured, monkeypatch, tmp_path):
    logger = log.get_logger()
    first = list(logger.handlers)
    log.configure_logging("ERROR")                                   # already configured: nothing changes
    assert logger.handlers == first and logger.level == logging.DEBUG
    monkeypatch.setenv("JIGSAW_LOG_LEVEL", "warning")
    monkeypatch.setenv("JIGSAW_LOG_RANK", "2")
    monkeypatch.setenv("JIGSAW_LOG_FORMAT", "json")
    monkeypatch.setenv("JIGSAW_LOG_DIR", str(tmp_path))
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("WORLD_SIZE", "4")
    log.configure_logging(install_excepthook=False, enable_faulthandler=False, capture_warnings=False, force=True)
    assert logger.level == logging.WARNING and log._state["print_rank"] == 2
    assert isinstance(logger.handlers[0].formatter, log._Json) and len(logger.handlers) == 2
    logger.handlers[0].stream = io.StringIO()
    log.warning("addressed to rank 2: not on the console of rank 1 ...")
    log.at(1).warning("for rank 1")
    for h in logger.handlers:
        h.flush()
    assert "for rank 1" in logger.handlers[0].stream.getvalue() and "addressed to rank 2" not in logger.handlers[0].stream.getvalue()
    in_file = [json.loads(row)["msg"] for row in (tmp_path / "rank_0001.log").read_text().splitlines()]
    assert len(in_file) == 2, "... but the per-rank file keeps every record of its rank"


def test_warnings_are_routed_through_the_logger(captured):
    logging.captureWarnings(False)          # an earlier configuration in this process may have left the hook half-installed
    log.configure_logging("DEBUG", as_json=True, install_excepthook=False, enable_faulthandler=False, capture_warnings=True, force=True)
    stream = io.StringIO()
    log.get_logger().handlers[0].stream = stream
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("always")
            warnings.warn("careful", UserWarning)
        assert "careful" in stream.getvalue()
    finally:
        logging.captureWarnings(False)
        wl = logging.getLogger("py.warnings")
        for h in list(wl.handlers):
            wl.removeHandler(h)


def test_uncaught_exceptions_are_logged_on_every_rank(captured, monkeypatch):
    monkeypatch.setattr(log, "_rank_world", lambda: (3, 4))
    calls = []
    monkeypatch.setattr(log, "_teardown", lambda: calls.append("teardown"))
    monkeypatch.setattr(sys, "excepthook", sys.__excepthook__)
    log._install_excepthook()
    hook = sys.excepthook
    log._install_excepthook()                                        # installing twice keeps one hook
    assert sys.excepthook is hook
    try:
        raise RuntimeError("fell over")
    except RuntimeError:
        hook(*sys.exc_info())
    got = captured()
    assert got[-1]["level"] == "CRITICAL" and "rank 3/4" in got[-1]["msg"] and "fell over" in got[-1]["exc"]
    assert calls == ["teardown"]
