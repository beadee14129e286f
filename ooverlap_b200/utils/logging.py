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
