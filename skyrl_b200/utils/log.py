"""Logger set-up: one format for every process, rank prefix, level from ``SKYRL_LOG_LEVEL``
(reference: skyrl/utils/log.py)."""

from __future__ import annotations

import logging
import os
import sys

_CONFIGURED = False


def setup_logging(level: str | None = None, rank: int | None = None) -> logging.Logger:
    global _CONFIGURED
    root = logging.getLogger("skyrl_b200")
    if _CONFIGURED:
        return root
    level = (level or os.environ.get("SKYRL_LOG_LEVEL", "INFO")).upper()
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    h = logging.StreamHandler(sys.stderr)
    h.setFormatter(logging.Formatter(f"%(asctime)s [rank {rank}] %(levelname)s %(name)s: %(message)s", "%H:%M:%S"))
    root.addHandler(h)
    root.setLevel(getattr(logging, level, logging.INFO))
    root.propagate = False
    _CONFIGURED = True
    return root


def get_logger(name: str = "skyrl_b200") -> logging.Logger:
    setup_logging()
    return logging.getLogger(name if name.startswith("skyrl_b200") else f"skyrl_b200.{name}")
