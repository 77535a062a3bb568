"""Named RNG streams so tensor-parallel shards draw different numbers and replicated tensors the same.

``model_parallel_manual_seed(seed)`` keeps the default stream at ``seed`` (identical across a TP group, used
for replicated parameters and data-parallel-consistent dropout) and registers
``model-parallel-rng`` = ``seed + 2718 + tp_rank`` and ``expert-parallel-rng`` =
``seed + 1024 + 100 * ep_rank + etp_rank``, the offsets Megatron uses, so weights initialised here match a
Megatron run with the same seed layout.  Works on CPU and CUDA generators.
"""
from __future__ import annotations

import contextlib
from typing import Dict

import torch

from . import state as ps

_MODEL_PARALLEL_RNG = 'model-parallel-rng'
_EXPERT_PARALLEL_RNG = 'expert-parallel-rng'
_DATA_PARALLEL_RNG = 'data-parallel-rng'


class RNGStatesTracker:

    def __init__(self):
        self.states: Dict[str, Dict[str, torch.Tensor]] = {}
        self.seeds = set()

    def reset(self):
        self.states.clear()
        self.seeds.clear()

    def _capture(self):
        st = {'cpu': torch.get_rng_state()}
        if torch.cuda.is_available():
            st['cuda'] = torch.cuda.get_rng_state()
        return st

    def _restore(self, st):
        torch.set_rng_state(st['cpu'])
        if 'cuda' in st and torch.cuda.is_available():
            torch.cuda.set_rng_state(st['cuda'])

    def add(self, name: str, seed: int):
        if name in self.states:
            raise RuntimeError(f'rng state {name} already exists')
        self.seeds.add(seed)
        orig = self._capture()
        torch.manual_seed(seed)
        self.states[name] = self._capture()
        self._restore(orig)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG):
        if name not in self.states:
            raise RuntimeError(f'rng state {name} was not added; call model_parallel_manual_seed first')
        orig = self._capture()
        self._restore(self.states[name])
        try:
            yield
        finally:
            self.states[name] = self._capture()
            self._restore(orig)


_TRACKER = RNGStatesTracker()


def get_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


def model_parallel_manual_seed(seed: int):
    _TRACKER.reset()
    torch.manual_seed(seed)
    c = ps.get_state().coords()
    _TRACKER.add(_DATA_PARALLEL_RNG, seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG, seed + 2718 + c['tp'])
    _TRACKER.add(_EXPERT_PARALLEL_RNG, seed + 1024 + 100 * c['ep'] + c['etp'])
