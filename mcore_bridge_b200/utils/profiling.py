"""Tracing helpers: NVTX ranges (no-ops without CUDA) and device-side timers built on CUDA events.

The reference only wraps a few ops in ``nvtx_range_push/pop``
(``src/mcore_bridge/model/modules/gated_delta_net.py:190-377``);
here every layer-level op can be wrapped with :func:`nvtx_range`, and :class:`DeviceTimers` accumulates per-name
device time (events are resolved lazily at ``summary()`` so measuring does not synchronise the step).
"""
from __future__ import annotations

import os
from collections import defaultdict
from contextlib import contextmanager
from typing import Dict, List, Tuple

import torch

_ENABLED = os.environ.get('MCB200_NVTX', '0') == '1'


def set_nvtx(enabled: bool):
    global _ENABLED
    _ENABLED = bool(enabled)


@contextmanager
def nvtx_range(name: str):
    if _ENABLED and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class DeviceTimers:

    def __init__(self):
        self._pairs: Dict[str, List[Tuple[torch.cuda.Event, torch.cuda.Event]]] = defaultdict(list)

    @contextmanager
    def time(self, name: str):
        if not torch.cuda.is_available():
            yield
            return
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        try:
            yield
        finally:
            e.record()
            self._pairs[name].append((s, e))

    def summary(self, reset: bool = True) -> Dict[str, Dict[str, float]]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = {}
        for name, pairs in self._pairs.items():
            ms = [s.elapsed_time(e) for s, e in pairs]
            out[name] = {'calls': len(ms), 'total_ms': sum(ms), 'mean_ms': sum(ms) / max(len(ms), 1)}
        if reset:
            self._pairs.clear()
        return out
