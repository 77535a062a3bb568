"""Python side of the fused compute+collective kernels (``csrc/comm/gemm_comm_sm100.cu``).

* :func:`all_gather_gemm` / :func:`all_gather_gemm_nn` — sequence-parallel all-gather fused into the consuming
  GEMM (column-parallel forward; row-parallel input-gradient).  Also returns the gathered operand, which the
  weight-gradient GEMM needs anyway.
* :func:`gemm_reduce_scatter` / :func:`gemm_reduce_scatter_nn` — GEMM fused with the reduce-scatter of its
  output (row-parallel forward; column-parallel input-gradient).

Each direction owns a symmetric workspace (``parallel/symm.py``): 64 KiB of flags followed by two data halves
used alternately (epoch parity).  ``enabled`` decides per call whether the fused path applies; otherwise the
caller uses ``torch.distributed``.  Set ``MCB200_FUSED_COMM=0`` to force the library path (the baseline).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from ..ops import _lib
from . import state as ps
from . import symm

FLAG_BYTES = 65536
_c_ll, _c_int = ctypes.c_longlong, ctypes.c_int
_ptr_cache: Dict[Tuple, ctypes.Array] = {}


def _on() -> bool:
    return os.environ.get('MCB200_FUSED_COMM', '1') != '0'


def enabled(x: torch.Tensor, weight: torch.Tensor, group_name: str) -> bool:
    """Fused path applies: bf16 CUDA tensors, 2..8 ranks on NVLink, row counts in whole 128-row blocks."""
    if not (_on() and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16):
        return False
    n = ps.get_world_size(group_name)
    if n < 2 or n > 8 or not symm.is_supported() or not _lib.available():
        return False
    return True


def _shapes_ok_ag(rows: int, K: int, N: int) -> bool:
    return rows % 128 == 0 and K % 8 == 0 and N % 8 == 0


def _shapes_ok_rs(M: int, n: int, K: int, N: int) -> bool:
    return M % (128 * n) == 0 and K % 8 == 0 and N % 8 == 0


def _ptr_array(ws: symm.SymmWorkspace, offset: int):
    key = (id(ws), offset)
    arr = _ptr_cache.get(key)
    if arr is None:
        arr = (ctypes.c_void_p * ws.world)(*[p + offset for p in ws.peer_ptrs])
        _ptr_cache[key] = arr
    return arr


def _workspace(group_name: str, tag: str, half_bytes: int) -> Tuple[symm.SymmWorkspace, int]:
    """Workspace with two halves of at least ``half_bytes``; returns (workspace, actual half size)."""
    key = symm._key(group_name, tag)
    ws = symm._WORKSPACES.get(key)
    if ws is not None:
        half = (ws.nbytes - FLAG_BYTES) // 2 // 1024 * 1024
        if half >= half_bytes:
            return ws, half
        # grow: nobody may still be reading the old segment
        torch.cuda.synchronize()
        torch.distributed.barrier(group=ps.get_group(group_name))
        del symm._WORKSPACES[key]
        _ptr_cache.clear()
    default = {'ag': 32 << 20, 'rs': 64 << 20}[tag]
    half = max(default, (half_bytes + 1023) // 1024 * 1024)
    ws = symm.get_workspace(group_name, FLAG_BYTES + 2 * half, tag)
    return ws, (ws.nbytes - FLAG_BYTES) // 2 // 1024 * 1024


def _ag(x2: torch.Tensor, b: torch.Tensor, b_inner: int, b_outer: int, b_mn: bool, n_out: int, k_in: int,
        bias: Optional[torch.Tensor], group_name: str):
    rows = x2.shape[0]
    ws, half = _workspace(group_name, 'ag', rows * k_in * 2)
    epoch = ws.next_epoch()
    off = FLAG_BYTES + (epoch & 1) * half
    shard = ws.view(off, (rows, k_in), torch.bfloat16)
    shard.copy_(x2)
    M = rows * ws.world
    gathered = torch.empty((M, k_in), dtype=torch.bfloat16, device=x2.device)
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x2.device)
    rc = _lib.lib().mcb_ag_gemm_bf16(
        _ptr_array(ws, off), _ptr_array(ws, 0), _lib.ptr(gathered), _lib.ptr(b), _c_ll(b_inner), _c_ll(b_outer),
        _c_ll(b.stride(0)), _c_int(int(b_mn)), _lib.ptr(out), _c_ll(out.stride(0)), _lib.ptr(bias), _c_int(M),
        _c_int(n_out), _c_int(k_in), _c_int(ws.world), _c_int(ws.rank), _c_int(epoch),
        _lib.ptr(_lib.status_word(x2.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_ag_gemm_bf16')
    return out, gathered


def all_gather_gemm(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], group_name: str):
    """``y[M, N] = gather(x2)[M, K] @ weight[N, K]^T (+ bias)``; returns ``(y, gathered_x)`` or ``None`` if the
    shape does not fit the kernel."""
    N, K = weight.shape
    if not _shapes_ok_ag(x2.shape[0], K, N) or not weight.is_contiguous():
        return None
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    return _ag(x2.contiguous(), weight, K, N, False, N, K, bias, group_name)


def all_gather_gemm_nn(dy2: torch.Tensor, weight: torch.Tensor, group_name: str):
    """``dx[M, K] = gather(dy2)[M, N] @ weight[N, K]``; returns ``(dx, gathered_dy)`` or ``None``."""
    N, K = weight.shape
    if not _shapes_ok_ag(dy2.shape[0], N, K) or not weight.is_contiguous():
        return None
    return _ag(dy2.contiguous(), weight, K, N, True, K, N, None, group_name)


def _rs(a2: torch.Tensor, b: torch.Tensor, b_inner: int, b_outer: int, b_mn: bool, n_out: int, k_in: int,
        group_name: str):
    M = a2.shape[0]
    n = ps.get_world_size(group_name)
    # staging is tile-major: one 64 KiB slot per 128 x 256 partial tile
    ws, half = _workspace(group_name, 'rs', (M // 128) * ((n_out + 255) // 256) * 65536)
    epoch = ws.next_epoch()
    off = FLAG_BYTES + (epoch & 1) * half
    out = torch.empty((M // n, n_out), dtype=torch.bfloat16, device=a2.device)
    rc = _lib.lib().mcb_gemm_rs_bf16(
        _lib.ptr(a2), _c_ll(a2.stride(0)), _lib.ptr(b), _c_ll(b_inner), _c_ll(b_outer), _c_ll(b.stride(0)),
        _c_int(int(b_mn)), _ptr_array(ws, off), _ptr_array(ws, 0), _lib.ptr(out), _c_ll(out.stride(0)), _c_int(M),
        _c_int(n_out), _c_int(k_in), _c_int(ws.world), _c_int(ws.rank), _c_int(epoch),
        _lib.ptr(_lib.status_word(a2.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_gemm_rs_bf16')
    return out


def gemm_reduce_scatter(x2: torch.Tensor, weight: torch.Tensor, group_name: str):
    """``y[M/n, N] = reduce_scatter(x2[M, K/n] @ weight[N, K/n]^T)``; ``None`` if the shape does not fit."""
    N, K = weight.shape
    n = ps.get_world_size(group_name)
    if not _shapes_ok_rs(x2.shape[0], n, K, N) or not weight.is_contiguous():
        return None
    if x2.stride(1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    return _rs(x2, weight, K, N, False, N, K, group_name)


def gemm_reduce_scatter_nn(dy2: torch.Tensor, weight: torch.Tensor, group_name: str):
    """``dx[M/n, K] = reduce_scatter(dy2[M, N/n] @ weight[N/n, K])``; ``None`` if the shape does not fit."""
    N, K = weight.shape
    n = ps.get_world_size(group_name)
    if not _shapes_ok_rs(dy2.shape[0], n, N, K) or not weight.is_contiguous() or N % 64:
        return None
    if dy2.stride(1) != 1 or dy2.stride(0) % 8:
        dy2 = dy2.contiguous()
    return _rs(dy2, weight, K, N, True, K, N, group_name)
