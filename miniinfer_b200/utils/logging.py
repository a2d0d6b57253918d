"""A small logger in the reference's format, ``LEVEL mm-dd HH:MM:SS [file:line] message``
(miniinfer/utils/logger.py:1-166), without colours.  Level from ``MINIINFER_B200_LOG`` (default WARNING)."""

from __future__ import annotations

import logging
import os
import sys

_configured = False


def get_logger(name: str) -> logging.Logger:
  global _configured
  if not _configured:
    handler = logging.StreamHandler(sys.stderr)
    handler.setFormatter(logging.Formatter("%(levelname)s %(asctime)s [%(filename)s:%(lineno)d] %(message)s",
                                           datefmt="%m-%d %H:%M:%S"))
    root = logging.getLogger("miniinfer_b200")
    root.addHandler(handler)
    root.setLevel(os.environ.get("MINIINFER_B200_LOG", "WARNING").upper())
    root.propagate = False
    _configured = True
  return logging.getLogger(name if name.startswith("miniinfer_b200") else f"miniinfer_b200.{name}")
