"""Logging set-up (``muse/utils/logger.py:30-82``): rank-tagged records, INFO on rank 0 and WARNING elsewhere."""
from __future__ import annotations

import logging
import sys
from typing import Optional

from .common import get_rank


def setup_logging(level: Optional[int] = None, log_file: Optional[str] = None) -> None:
    rank = get_rank()
    level = level if level is not None else (logging.INFO if rank == 0 else logging.WARNING)
    handlers = [logging.StreamHandler(sys.stdout)]
    if log_file and rank == 0:
        handlers.append(logging.FileHandler(log_file))
    logging.basicConfig(level=level, format=f"%(asctime)s [rank {rank}] %(levelname)s %(name)s: %(message)s",
                        handlers=handlers, force=True)


def get_logger(name: str = "ksa_b200") -> logging.Logger:
    return logging.getLogger(name)
