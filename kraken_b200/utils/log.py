"""Logging set-up of the package.

The reference logs through LOG_DEBUG / LOG_INFO / LOG_WARNING / LOG_ERROR macros to stdout as
``[thread id] timestamp file:line:message`` with a compile-time level (kraken/common/log.h:105-128,
kraken/common/log.cc:6-10).  Here the ``kraken_b200`` logger prints the same shape with the rank in
place of the thread id and takes its level at run time from ``KRAKEN_LOG_LEVEL``
(debug / info / warning / error; default warning).  ``configure()`` is idempotent and is called by
``kraken.pytorch.initialize`` and by the server executables.
"""
from __future__ import annotations

import logging
import os
import sys

_LEVELS = {"debug": logging.DEBUG, "info": logging.INFO, "warning": logging.WARNING, "warn": logging.WARNING,
           "error": logging.ERROR}
_configured = False


class _RankFilter(logging.Filter):
    def filter(self, record: logging.LogRecord) -> bool:
        record.rank = os.environ.get("RANK", "0")
        return True


def configure(level: str | None = None, stream=None) -> logging.Logger:
    """Installs the handler once; a later call only changes the level when one is given."""
    global _configured
    log = logging.getLogger("kraken_b200")
    name = (level or os.environ.get("KRAKEN_LOG_LEVEL", "warning")).lower()
    if not _configured:
        handler = logging.StreamHandler(stream or sys.stdout)
        handler.setFormatter(logging.Formatter("[%(rank)s] %(asctime)s.%(msecs)03d %(filename)s:%(lineno)d:%(message)s",
                                               datefmt="%Y-%m-%d %H:%M:%S"))
        handler.addFilter(_RankFilter())
        log.addHandler(handler)
        log.propagate = False
        _configured = True
        log.setLevel(_LEVELS.get(name, logging.WARNING))
    elif level is not None:
        log.setLevel(_LEVELS.get(name, logging.WARNING))
    return log
