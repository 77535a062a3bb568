"""Symmetric (peer-mapped) workspaces for the fused compute+collective kernels.

A workspace is one allocation of the same size on every rank of a process group, mapped into every peer's
address space, plus a signal pad of 32-bit flags.  Allocation and handle exchange go through
``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged over the group's store — plumbing only);
everything that moves data is in-tree kernels that receive the raw peer pointers.

Protocol state kept here:
* ``epoch`` — incremented by every fused call on the workspace; kernels publish / wait for flags carrying the
  epoch, so flags never need clearing between calls.
* double buffering by epoch parity: a rank overwrites the half used two calls ago.  Observing every peer's
  "ready" flag for call ``e+1`` proves the peer finished call ``e`` (stream order on the peer), hence finished
  reading this rank's half ``e``; that half is next written for call ``e+2``.  No extra hand-shake is needed as
  long as every rank issues the same sequence of fused calls on a workspace (SPMD).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from . import state as ps

_WORKSPACES: Dict[str, 'SymmWorkspace'] = {}
SIGNAL_WORDS = 4096  # uint32 flags per rank that this module hands out (the pad itself may be larger)


@dataclass
class SymmWorkspace:
    group_name: str
    world: int
    rank: int
    nbytes: int
    buffer: torch.Tensor                 # uint8 [nbytes], this rank's segment
    peer_ptrs: List[int]                 # device pointers of every rank's segment, indexed by group rank
    signal_ptrs: List[int]               # device pointers of every rank's signal pad
    multicast_ptr: int                   # 0 when NVLS multicast is not available
    handle: object = None
    epoch: int = 0
    ptr_table: Optional[torch.Tensor] = None     # int64 [2, world] on device: buffer ptrs, signal ptrs

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = int(torch.tensor(shape).prod().item()) * torch.empty((), dtype=dtype).element_size()
        assert offset % 16 == 0 and offset + n <= self.nbytes, (offset, n, self.nbytes)
        return self.buffer[offset:offset + n].view(dtype).view(*shape)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


def is_supported() -> bool:
    if not torch.cuda.is_available() or not dist.is_available() or not dist.is_initialized():
        return False
    try:
        import importlib
        importlib.import_module('torch.distributed._symmetric_memory')
        return dist.get_backend() == 'nccl'
    except Exception:
        return False


def _key(group_name: str, tag: str) -> str:
    # the member ranks are part of the identity: after the parallel state is rebuilt with other groups of the same
    # name, an old workspace (mapped to other peers) must not be handed out
    return f"{group_name}:{','.join(map(str, ps.get_group_ranks(group_name)))}:{tag}"


def get_workspace(group_name: str, nbytes: int, tag: str = 'default') -> SymmWorkspace:
    """Returns (allocating or growing on first use — a collective call over the group) the named workspace."""
    key = _key(group_name, tag)
    ws = _WORKSPACES.get(key)
    if ws is not None and ws.nbytes >= nbytes:
        return ws
    import torch.distributed._symmetric_memory as symm_mem
    group = ps.get_group(group_name)
    assert group is not None, f'group {group_name} has a single rank: no symmetric workspace needed'
    nbytes = (nbytes + (1 << 21) - 1) >> 21 << 21  # 2 MiB granularity (VMM page)
    dev = torch.device('cuda', torch.cuda.current_device())
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
    handle = symm_mem.rendezvous(buf, group=group)
    world, rank = handle.world_size, handle.rank
    peer_ptrs = [int(p) for p in handle.buffer_ptrs]
    signal_ptrs = [int(p) for p in handle.signal_pad_ptrs]
    mc = int(getattr(handle, 'multicast_ptr', 0) or 0)
    buf.zero_()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    table = torch.tensor([peer_ptrs, signal_ptrs], dtype=torch.int64, device=dev)
    ws = SymmWorkspace(group_name, world, rank, nbytes, buf, peer_ptrs, signal_ptrs, mc, handle, 0, table)
    _WORKSPACES[key] = ws
    return ws


def release_workspace(group_name: str, tag: str) -> None:
    """Forgets a workspace; its memory goes back once the last tensor viewing it is gone (on every rank)."""
    _WORKSPACES.pop(_key(group_name, tag), None)


def free_all():
    _WORKSPACES.clear()
