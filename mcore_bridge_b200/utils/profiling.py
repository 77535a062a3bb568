"""Tracing helpers: NVTX ranges (no-ops without CUDA) and device-side timers built on CUDA events.

The reference only wraps a few ops in ``nvtx_range_push/pop``
(``src/mcore_bridge/model/modules/gated_delta_net.py:190-377``);
here the layer-level ops (attention block: ``qkv`` / ``qk_norm_rope`` / ``core_attention`` / ``linear_proj``; the
gated-DeltaNet stages; ``mlp`` / ``moe``; the trainer's ``forward_backward`` / ``optimizer``) sit inside
:func:`nvtx_range`, and :class:`DeviceTimers` accumulates per-name device time (events are resolved lazily at
``summary()`` so measuring does not synchronise the step).
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


class _NoRange:
    """What :func:`nvtx_range` returns while tracing is off: entering and leaving it does nothing."""
    __slots__ = ()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _Range:
    __slots__ = ('name',)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


_NO_RANGE = _NoRange()


def nvtx_range(name: str):
    """``with nvtx_range('core_attention'): ...`` — an NVTX range when tracing is on (``MCB200_NVTX=1`` or
    :func:`set_nvtx`) and CUDA is present, otherwise a shared do-nothing object (no allocation on the hot path)."""
    if _ENABLED and torch.cuda.is_available():
        return _Range(name)
    return _NO_RANGE


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
