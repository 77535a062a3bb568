"""Data-parallel collectives of the distributed optimizer on the in-tree peer-memory kernels
(``csrc/comm/dp_collectives.cu``): the fp32 gradient reduce-scatter and the parameter all-gather read the other
ranks' flat buffers directly over NVLink instead of going through ``torch.distributed``.

A flat buffer that takes part lives in a symmetric workspace (``parallel/symm.py``): ``FLAG_BYTES`` of epoch flags
followed by the data.  ``usable`` decides once per buffer; ``MCB200_FUSED_DP=0`` forces the library path (the
baseline the kernels are measured against).
"""
from __future__ import annotations

import ctypes
import itertools
import os
from typing import Tuple

import torch

from ..ops import _lib
from . import state as ps
from . import symm

FLAG_BYTES = 65536
_c_ll, _c_int = ctypes.c_longlong, ctypes.c_int
_counter = itertools.count()
CTAS = int(os.environ.get('MCB200_DP_CTAS', '0'))   # 0: the launcher's default


def usable(group_name: str, device) -> bool:
    """2..8 ranks of one node on NCCL, CUDA buffers, the in-tree library loaded."""
    if os.environ.get('MCB200_FUSED_DP', '1') == '0' or torch.device(device).type != 'cuda':
        return False
    n = ps.get_world_size(group_name)
    if n < 2 or n > 8 or not symm.is_supported() or not _lib.available():
        return False
    return torch.distributed.get_world_size() <= torch.cuda.device_count()      # peers must be P2P-mapped


def allocate(group_name: str, numel: int, dtype) -> Tuple[symm.SymmWorkspace, torch.Tensor]:
    """A zeroed flat tensor of ``numel`` elements that every rank of the group can read (collective call)."""
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    ws = symm.get_workspace(group_name, FLAG_BYTES + nbytes, f'dp{next(_counter)}')
    return ws, ws.view(FLAG_BYTES, (numel,), dtype)


def _ptrs(ws: symm.SymmWorkspace, offset: int):
    return (ctypes.c_void_p * ws.world)(*[p + offset for p in ws.peer_ptrs])


def reduce_scatter_(ws: symm.SymmWorkspace, data: torch.Tensor, start: int, end: int, scale: float = 1.0) -> None:
    """In place on the current stream: elements ``[start, end)`` of ``data`` (the workspace's flat fp32 tensor) are a
    bucket; this rank's ``1/world`` slice of it becomes the sum over all ranks (times ``scale``)."""
    assert data.dtype == torch.float32 and (end - start) % ws.world == 0
    shard_bytes = (end - start) // ws.world * 4
    rc = _lib.lib().mcb_dp_reduce_scatter_f32(
        _ptrs(ws, FLAG_BYTES), _ptrs(ws, 0), _c_ll(start * 4), _c_ll(shard_bytes), _c_int(ws.world), _c_int(ws.rank),
        _c_int(ws.next_epoch()), ctypes.c_float(scale), _c_int(CTAS), _lib.ptr(_lib.status_word(data.device)),
        _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_dp_reduce_scatter_f32')


def all_gather_(ws: symm.SymmWorkspace, data: torch.Tensor, start: int, end: int) -> None:
    """In place on the current stream: every rank's slice of the bucket ``[start, end)`` is copied into this rank's
    buffer at its final position."""
    es = data.element_size()
    assert (end - start) % ws.world == 0
    shard_bytes = (end - start) // ws.world * es
    rc = _lib.lib().mcb_dp_all_gather(
        _ptrs(ws, FLAG_BYTES), _ptrs(ws, 0), _c_ll(start * es), _c_ll(shard_bytes), _c_int(ws.world), _c_int(ws.rank),
        _c_int(ws.next_epoch()), _c_int(CTAS), _lib.ptr(_lib.status_word(data.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_dp_all_gather')
