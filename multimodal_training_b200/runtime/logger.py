"""Process-wide logging: console plus a shared append-mode file tagged with the PID.

Same contract as the reference (python/ray/logger.py:15-94): idempotent ``setup_logging``; the file
path comes from ``RAY_TRAIN_LOG_FILE`` (``MMT_TRAIN_LOG_FILE`` also accepted) or defaults to
``/tmp/ray_train.log``; console lines are ``%(asctime)s - %(message)s``.
"""
from __future__ import annotations

import logging
import os
import sys

_CONFIGURED = False
DEFAULT_LOG_FILE = "/tmp/ray_train.log"


def log_file_path() -> str:
    return os.environ.get("MMT_TRAIN_LOG_FILE") or os.environ.get("RAY_TRAIN_LOG_FILE") or DEFAULT_LOG_FILE


def setup_logging(level: int = logging.INFO, force: bool = False, log_file: str | None = None) -> logging.Logger:
    global _CONFIGURED
    root = logging.getLogger()
    if _CONFIGURED and not force:
        return root
    for h in list(root.handlers):
        root.removeHandler(h)
    root.setLevel(level)
    console = logging.StreamHandler(sys.stdout)
    console.setFormatter(logging.Formatter("%(asctime)s - %(message)s"))
    root.addHandler(console)
    path = log_file or log_file_path()
    try:
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        fh = logging.FileHandler(path, mode="a")
        fh.setFormatter(logging.Formatter(f"%(asctime)s - [pid {os.getpid()}] %(levelname)s - %(message)s"))
        root.addHandler(fh)
    except OSError:
        root.warning("cannot open log file %s; logging to console only", path)
    os.environ.setdefault("KINETO_LOG_LEVEL", "5")
    _CONFIGURED = True
    return root
