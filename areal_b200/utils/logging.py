"""Coloured per-component loggers with an optional shared file handler
(reference: ``areal/utils/logging.py``)."""
from __future__ import annotations

import logging
import os
import sys
from typing import Optional

_FMT = "%(asctime)s.%(msecs)03d %(name)s %(levelname)s: %(message)s"
_DATE = "%Y%m%d-%H:%M:%S"
_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[35m"}
_RESET = "\033[0m"
_configured = False
_file_handler: Optional[logging.Handler] = None


class _ColorFormatter(logging.Formatter):
    def format(self, record):
        msg = super().format(record)
        if sys.stderr.isatty():
            return f"{_COLORS.get(record.levelname, '')}{msg}{_RESET}"
        return msg


def _configure():
    global _configured
    if _configured:
        return
    root = logging.getLogger("areal_b200")
    root.setLevel(os.environ.get("AREAL_LOG_LEVEL", "INFO").upper())
    h = logging.StreamHandler(sys.stderr)
    h.setFormatter(_ColorFormatter(_FMT, _DATE))
    root.addHandler(h)
    root.propagate = False
    _configured = True


def getLogger(name: Optional[str] = None) -> logging.Logger:
    _configure()
    return logging.getLogger("areal_b200" if not name else f"areal_b200.{name}")


def setup_file_logging(log_dir: str, filename: str = "main.log") -> str:
    """Adds one file handler shared by all component loggers."""
    global _file_handler
    _configure()
    os.makedirs(log_dir, exist_ok=True)
    path = os.path.join(log_dir, filename)
    root = logging.getLogger("areal_b200")
    if _file_handler is not None:
        root.removeHandler(_file_handler)
    _file_handler = logging.FileHandler(path)
    _file_handler.setFormatter(logging.Formatter(_FMT, _DATE))
    root.addHandler(_file_handler)
    return path
