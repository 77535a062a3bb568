"""Host-side liveness: every rank writes a heartbeat between steps, any rank can list the ones that stopped.

Failure detection never relies on a GPU fault: a rank that died, hung on the host or left shows up as a stale
heartbeat (or as a process-group timeout on the next collective), and the survivors learn of it before their next
launch.  The store is a directory of small files, which also works across nodes on a shared filesystem; a
``torch.distributed`` store could be dropped in with the same interface.
"""
from __future__ import annotations

import json
import os
import time
from typing import List, Optional


class HeartbeatMonitor:

    def __init__(self, directory: str, rank: int, world: int, timeout_s: float = 60.0):
        self.dir, self.rank, self.world, self.timeout_s = directory, rank, world, timeout_s
        os.makedirs(directory, exist_ok=True)

    def _path(self, r: int) -> str:
        return os.path.join(self.dir, f'rank{r:05d}.json')

    def beat(self, step: int, status: str = 'ok') -> None:
        tmp = self._path(self.rank) + '.tmp'
        with open(tmp, 'w') as f:
            json.dump({'t': time.time(), 'step': step, 'status': status}, f)
        os.replace(tmp, self._path(self.rank))

    def read(self, r: int) -> Optional[dict]:
        try:
            with open(self._path(r)) as f:
                return json.load(f)
        except (FileNotFoundError, json.JSONDecodeError):
            return None

    def dead_ranks(self, now: Optional[float] = None, missing_is_dead: bool = True) -> List[int]:
        """Ranks whose heartbeat is stale or reports a failure.  A rank that has not written one yet counts as dead
        unless ``missing_is_dead`` is False (the check at the start of a run, before everybody's first beat)."""
        now = time.time() if now is None else now
        dead = []
        for r in range(self.world):
            hb = self.read(r)
            if hb is None:
                if missing_is_dead:
                    dead.append(r)
            elif now - hb['t'] > self.timeout_s or hb.get('status') != 'ok':
                dead.append(r)
        return dead


class RankFailure(RuntimeError):
    """Raised on a surviving rank, on the host and before its next launch, when other ranks stopped beating."""

    def __init__(self, ranks: List[int]):
        super().__init__(f'ranks {ranks} stopped answering (stale or failed heartbeat)')
        self.ranks = ranks
