"""Rank-aware logger with ``info_once`` / ``warning_once``.

Parity: reference ``src/mcore_bridge/utils/logger.py:25-80`` (level from ``LOG_LEVEL``; only the
local master logs below ERROR).
"""
from __future__ import annotations

import logging
import os
from types import MethodType
from typing import Optional

_initialised = {}
_once_cache = set()


def _is_local_master() -> bool:
    return int(os.getenv('LOCAL_RANK', -1)) in {-1, 0}


def _info_once(self, msg, *args, hash_id=None, **kwargs):
    key = ('info', hash_id or msg)
    if key in _once_cache:
        return
    _once_cache.add(key)
    self.info(msg, *args, **kwargs)


def _warning_once(self, msg, *args, hash_id=None, **kwargs):
    key = ('warning', hash_id or msg)
    if key in _once_cache:
        return
    _once_cache.add(key)
    self.warning(msg, *args, **kwargs)


def get_logger(log_level: Optional[int] = None, name: str = 'mcore_bridge_b200'):
    if log_level is None:
        log_level = getattr(logging, os.getenv('LOG_LEVEL', 'INFO').upper(), logging.INFO)
    logger = logging.getLogger(name)
    if name in _initialised:
        return logger
    logger.propagate = False
    handler = logging.StreamHandler()
    handler.setFormatter(logging.Formatter('[%(levelname)s:%(name)s] %(message)s'))
    logger.addHandler(handler)
    level = log_level if _is_local_master() else logging.ERROR
    handler.setLevel(level)
    logger.setLevel(level)
    logger.info_once = MethodType(_info_once, logger)
    logger.warning_once = MethodType(_warning_once, logger)
    _initialised[name] = True
    return logger
