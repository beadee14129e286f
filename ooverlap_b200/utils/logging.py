"""Package logger with the reference's level names.

Capability parity: include/ooverlap/system/logging.h:22-147 (compile-time
levels FATAL..TRACE with file:line); here the level is a run-time setting
(OOB_LOG_LEVEL) of a standard ``logging`` logger.
"""
from __future__ import annotations

import logging
import os

_LEVELS = {"fatal": logging.CRITICAL, "error": logging.ERROR, "warning": logging.WARNING, "warn": logging.WARNING,
           "info": logging.INFO, "debug": logging.DEBUG, "trace": 5}

logger = logging.getLogger("ooverlap_b200")


def setup(level: str | None = None) -> logging.Logger:
    name = (level or os.environ.get("OOB_LOG_LEVEL", "warning")).lower()
    logger.setLevel(_LEVELS.get(name, logging.WARNING))
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("[oob %(levelname)s %(filename)s:%(lineno)d] %(message)s"))
        logger.addHandler(h)
        logger.propagate = False
    return logger


setup()

_NATIVE_TO_PY = {0: logging.ERROR, 1: logging.WARNING, 2: logging.INFO, 3: logging.DEBUG}
_sink_ref = None  # keeps the ctypes callback alive for as long as the library may call it


def set_native_log_level(level) -> None:
    """Level of the native runtime's own records (0 / "error", 1 / "warn", 2 / "info", 3 / "debug"); the environment
    variable OOB_LOG_LEVEL sets both this and the Python logger at start-up."""
    from .. import _lib
    names = {"fatal": 0, "error": 0, "warn": 1, "warning": 1, "info": 2, "debug": 3, "trace": 3}
    code = names[level.lower()] if isinstance(level, str) else int(level)
    _lib.check(_lib.lib().oob_set_log_level(code))


def forward_native_logs(enable: bool = True) -> None:
    """Routes the native runtime's records (communicator set-up, NVLS refusals, device timeouts, IPC cache traffic)
    into this package's ``logging`` logger instead of stderr.  The callback may run on any thread that calls into the
    library; switch it off again before interpreter shutdown if other threads may still be inside the library."""
    global _sink_ref
    from .. import _lib
    if not enable:
        _lib.check(_lib.lib().oob_set_log_sink(_lib.LOG_SINK()))
        _sink_ref = None
        return

    def sink(level: int, message: bytes) -> None:
        logger.log(_NATIVE_TO_PY.get(level, logging.INFO), "native: %s", message.decode(errors="replace"))

    _sink_ref = _lib.LOG_SINK(sink)
    _lib.check(_lib.lib().oob_set_log_sink(_sink_ref))
