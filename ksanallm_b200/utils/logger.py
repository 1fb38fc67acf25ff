"""Python face of the native logger (csrc/engine/logger.{h,cpp}): one sink for the C++ runtime and the Python layers.

Level and target come from the environment like the reference's logger (src/ksana_llm/utils/logger.h:15-40):
``KLLM_LOG_LEVEL`` = DEBUG | INFO | WARNING | ERROR | FATAL (default INFO), ``KLLM_LOG_FILE`` (default
``log/ksana_llm.log``; ``stderr`` writes to standard error). ``install_logging_handler()`` also routes Python's
``logging`` records (uvicorn, the serving layer) to that sink.
"""
from __future__ import annotations

import logging
import os
import sys

from . import native_engine as ne

DEBUG, INFO, WARNING, ERROR, FATAL = 0, 1, 2, 3, 4


def _emit(level: int, msg: str, depth: int = 2) -> None:
    if not ne.log_enabled(level):
        return
    f = sys._getframe(depth)
    ne.log_message(level, os.path.basename(f.f_code.co_filename), f.f_lineno, str(msg))


def debug(msg) -> None:
    _emit(DEBUG, msg)


def info(msg) -> None:
    _emit(INFO, msg)


def warning(msg) -> None:
    _emit(WARNING, msg)


def error(msg) -> None:
    _emit(ERROR, msg)


def fatal(msg) -> None:
    _emit(FATAL, msg)


def set_level(name: str) -> None:
    ne.set_log_level(name.upper())


def set_file(path: str) -> None:
    ne.set_log_file(path)


def log_file() -> str:
    return ne.log_file()


class NativeLogHandler(logging.Handler):
    """Forwards Python ``logging`` records to the native sink, keeping their source location."""

    _MAP = ((logging.CRITICAL, FATAL), (logging.ERROR, ERROR), (logging.WARNING, WARNING), (logging.INFO, INFO))

    def emit(self, record: logging.LogRecord) -> None:
        level = DEBUG
        for py, ours in self._MAP:
            if record.levelno >= py:
                level = ours
                break
        if ne.log_enabled(level):
            try:
                text = record.getMessage()
            except Exception:  # noqa: BLE001 - a bad format string must not raise from a log call
                text = str(record.msg)
            ne.log_message(level, f"{record.name}:{os.path.basename(record.pathname)}", record.lineno, text)


_installed = False


def install_logging_handler(logger_name: str = "") -> None:
    """Route Python ``logging`` (root logger by default) to the native sink, once."""
    global _installed
    if _installed:
        return
    _installed = True
    lg = logging.getLogger(logger_name)
    lg.addHandler(NativeLogHandler())
    py_level = {DEBUG: logging.DEBUG, INFO: logging.INFO, WARNING: logging.WARNING, ERROR: logging.ERROR,
                FATAL: logging.CRITICAL}[ne.log_level()]
    if lg.level == logging.NOTSET or lg.level > py_level:
        lg.setLevel(py_level)
