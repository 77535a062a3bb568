"""Collective-order checker: a debugging aid that turns "the ranks of a group issued different collectives" from a hang
into an exception that names the group, the position in the sequence and what each rank tried to do.

While installed (``with CollectiveOrderChecker(): ...``, or ``MCB200_CHECK_COLLECTIVES=1`` in the trainer), every
``torch.distributed`` collective first publishes a signature (operation, element count, dtype) under a key made of the
group's member ranks and a per-group sequence number in the job's rendezvous store, then reads the signatures of the
other members with a time limit. A different signature raises :class:`CollectiveMismatch` on every rank that sees it;
a member that never arrives raises :class:`CollectiveTimeout` on the ones waiting. Nothing runs on a device: the
comparison happens on the host before the collective is launched, so a diverged rank never leaves a kernel waiting for
its peers. It costs a store round trip per collective and is meant for reproducing a hang, not for production steps.

The reference has no such facility: its lock-step weight export relies on flag all-reduces to keep ranks on the same
branch (``src/mcore_bridge/bridge/gpt_bridge.py:358-382,469-472``).
"""
from __future__ import annotations

import os
from datetime import timedelta
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class CollectiveMismatch(RuntimeError):
    pass


class CollectiveTimeout(RuntimeError):
    pass


def _meta(t) -> str:
    if isinstance(t, torch.Tensor):
        return f'{t.numel()}x{str(t.dtype).replace("torch.", "")}'
    if isinstance(t, (list, tuple)):
        return '[' + ','.join(_meta(x) for x in t) + ']'
    return type(t).__name__


# name -> positions of the tensor arguments that take part in the signature
_OPS = {
    'all_reduce': (0,), 'broadcast': (0,), 'all_gather_into_tensor': (0, 1), 'reduce_scatter_tensor': (0, 1),
    'all_to_all_single': (0, 1), 'all_gather': (0, 1), 'reduce_scatter': (0, 1), 'barrier': (),
    'all_gather_object': (),
}


class CollectiveOrderChecker:

    def __init__(self, timeout_s: float = 30.0, store=None):
        self.timeout = timedelta(seconds=timeout_s)
        self._store = store
        self._seq: Dict[tuple, int] = {}
        self._orig = {}

    # ------------------------------------------------------------------ install / remove
    def __enter__(self):
        return self.install()

    def __exit__(self, *exc):
        self.remove()
        return False

    def install(self):
        if self._store is None:
            self._store = dist.distributed_c10d._get_default_store()
        for name, positions in _OPS.items():
            orig = getattr(dist, name, None)
            if orig is None:
                continue
            self._orig[name] = orig
            setattr(dist, name, self._wrap(name, orig, positions))
        return self

    def remove(self):
        for name, orig in self._orig.items():
            setattr(dist, name, orig)
        self._orig.clear()

    def _wrap(self, name, orig, positions):
        def checked(*args, **kwargs):
            group = kwargs.get('group')
            if group is None:
                for a in args:
                    if isinstance(a, dist.ProcessGroup):
                        group = a
            sig = name + '(' + ','.join(_meta(args[i]) for i in positions if i < len(args)) + ')'
            if name == 'all_to_all_single' and args and isinstance(args[0], torch.Tensor):
                # ranks legitimately exchange different amounts (expert-parallel dispatch): compare the dtype only
                sig = f'{name}({str(args[0].dtype).replace("torch.", "")})'
            if name == 'broadcast':
                sig += f' src={kwargs.get("src", args[1] if len(args) > 1 else None)}'
            self.check(sig, group)
            return orig(*args, **kwargs)
        checked.__wrapped__ = orig
        return checked

    # ------------------------------------------------------------------ the check itself
    def check(self, signature: str, group: Optional[dist.ProcessGroup] = None):
        ranks: List[int] = dist.get_process_group_ranks(group) if group is not None else \
            list(range(dist.get_world_size()))
        me = dist.get_rank()
        if me not in ranks or len(ranks) < 2:
            return
        gid = tuple(ranks)
        seq = self._seq.get(gid, 0)
        self._seq[gid] = seq + 1
        base = f'mcb200/cc/{"-".join(map(str, ranks))}/{seq}'
        self._store.set(f'{base}/{me}', signature)
        for r in ranks:
            if r == me:
                continue
            key = f'{base}/{r}'
            try:
                self._store.wait([key], self.timeout)
            except Exception as e:                      # the store raises on its time limit
                raise CollectiveTimeout(f'rank {r} did not reach collective #{seq} of group {list(ranks)} within '
                                        f'{self.timeout.total_seconds():.0f} s; rank {me} is at {signature}') from e
            other = self._store.get(key).decode()
            if other != signature:
                raise CollectiveMismatch(f'collective #{seq} of group {list(ranks)}: rank {me} issues {signature}, '
                                         f'rank {r} issues {other}')


def enabled_by_env() -> bool:
    return os.environ.get('MCB200_CHECK_COLLECTIVES', '0') == '1'
