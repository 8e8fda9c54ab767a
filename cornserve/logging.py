"""Logging helpers: ``LEVEL time [name:line] message`` on stderr, level from ``CORNSERVE_LOG_LEVEL``
(same convention as the reference, python/cornserve/logging.py:12-43)."""

from __future__ import annotations

import logging
import os
import sys


def get_logger(name: str, adapters: list | None = None) -> logging.Logger | logging.LoggerAdapter:
    logger = logging.getLogger(name)
    if not logger.handlers:
        level = os.environ.get("CORNSERVE_LOG_LEVEL", "INFO").upper()
        handler = logging.StreamHandler(sys.stderr)
        handler.setFormatter(logging.Formatter("%(levelname)s %(asctime)s [%(name)s:%(lineno)d] %(message)s"))
        logger.addHandler(handler)
        logger.setLevel(level)
        logger.propagate = False
    out: logging.Logger | logging.LoggerAdapter = logger
    for make in adapters or []:
        out = make(out)
    return out


class SidecarAdapter(logging.LoggerAdapter):
    """Prefixes every record with the sidecar rank."""

    def __init__(self, logger, rank: int):
        super().__init__(logger, {})
        self.rank = rank

    def process(self, msg, kwargs):
        return f"Sidecar {self.rank}: {msg}", kwargs
