"""Context-parallel attention.

Every CP rank holds, for each packed sequence, the zig-zag chunks ``r`` and ``2cp-1-r`` (``split_cp_inputs``), which
balances causal work.  Attention of the local queries needs all keys/values that precede them:

* keys/values are all-gathered over the CP group (differentiable: the backward is a reduce-scatter of dK/dV) and
  put back into original token order;
* each local chunk becomes one entry of a variable-length batch whose query block is the chunk and whose key block is
  the sequence prefix ending with the chunk (bottom-right aligned causal attention), so the regular varlen attention
  op computes it.

This is the all-gather formulation (``cp_comm_type='allgather'``) of the exchange the reference reaches through
TransformerEngine's ring (``cp_comm_type='p2p'``, ``src/mcore_bridge/config/model_config.py:240``); the results are
identical, the ring variant only overlaps the transfer with compute.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops.attention import attention_ref
from ..utils.megatron_utils import cp_gather_index
from . import state as ps


class _AllGatherTokens(torch.autograd.Function):
    """``[T_local, ...]`` -> ``[cp * T_local, ...]`` rank-major; backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        n = ps.get_world_size(group_name)
        out = torch.empty((n * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=ps.get_group(group_name))
        return out

    @staticmethod
    def backward(ctx, g):
        n = ps.get_world_size(ctx.group_name)
        g = g.contiguous()
        if g.is_cuda:
            out = torch.empty((g.shape[0] // n, *g.shape[1:]), dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, group=ps.get_group(ctx.group_name))
            return out, None
        tmp = g.clone()
        dist.all_reduce(tmp, group=ps.get_group(ctx.group_name))
        r = ps.get_rank_in(ctx.group_name)
        c = g.shape[0] // n
        return tmp[r * c:(r + 1) * c].contiguous(), None


def local_chunk_layout(cu_seqlens: torch.Tensor, cp: int, rank: int) -> List[Tuple[int, int, int]]:
    """For this rank: ``(local_start, global_start, length)`` of every chunk in local token order."""
    bounds = [int(x) for x in cu_seqlens.tolist()]
    out, loc = [], 0
    for s, e in zip(bounds[:-1], bounds[1:]):
        c = (e - s) // (2 * cp)
        out.append((loc, s + rank * c, c))
        out.append((loc + c, s + (2 * cp - rank - 1) * c, c))
        loc += 2 * c
    return out


def gather_to_stream_order(x: torch.Tensor, ctx) -> torch.Tensor:
    """``[T_local, ...]`` on every CP rank -> ``[cp * T_local, ...]`` in the order of the original token stream
    (differentiable: the backward reduce-scatters)."""
    cp = ps.get_world_size('cp')
    full = _AllGatherTokens.apply(x, 'cp')
    index = cp_gather_index(ctx.cu_seqlens, x.shape[0] * cp, cp).to(x.device)
    return full.index_select(0, index)


def stream_index_of_local_tokens(ctx, device) -> torch.Tensor:
    """Position in the original token stream of every token this CP rank holds, in local order."""
    parts = [torch.arange(g0, g0 + c, device=device)
             for _, g0, c in local_chunk_layout(ctx.cu_seqlens, ps.get_world_size('cp'), ps.get_rank_in('cp')) if c]
    return torch.cat(parts)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx, scale: Optional[float] = None,
                   window=None, sinks=None) -> torch.Tensor:
    """``q/k/v`` hold this rank's tokens ``[T_local, heads, d]``; returns ``[T_local, nq, dv]``."""
    cp = ps.get_world_size('cp')
    rank = ps.get_rank_in('cp')
    cu = ctx.cu_seqlens
    T_local = q.shape[0]
    kg = _AllGatherTokens.apply(k, 'cp')
    vg = _AllGatherTokens.apply(v, 'cp')
    index = cp_gather_index(cu, T_local * cp, cp).to(q.device)
    k_full, v_full = kg.index_select(0, index), vg.index_select(0, index)      # original token order
    bounds = [int(x) for x in cu.tolist()]
    seq_of = {}
    for s, e in zip(bounds[:-1], bounds[1:]):
        seq_of[s] = e
    chunks = local_chunk_layout(cu, cp, rank)
    # one varlen entry per chunk: queries = the chunk, keys = its sequence from the start up to the chunk's end
    q_parts, k_parts, v_parts, cu_q, cu_k = [], [], [], [0], [0]
    starts = sorted(seq_of)
    import bisect
    for loc, g0, c in chunks:
        if c == 0:
            continue
        s0 = starts[bisect.bisect_right(starts, g0) - 1]
        q_parts.append(q[loc:loc + c])
        k_parts.append(k_full[s0:g0 + c])
        v_parts.append(v_full[s0:g0 + c])
        cu_q.append(cu_q[-1] + c)
        cu_k.append(cu_k[-1] + (g0 + c - s0))
    qq, kk, vv = torch.cat(q_parts), torch.cat(k_parts), torch.cat(v_parts)
    cuq = torch.tensor(cu_q, dtype=torch.int32, device=q.device)
    cuk = torch.tensor(cu_k, dtype=torch.int32, device=q.device)
    if q.is_cuda and sinks is None and q.dtype in (torch.bfloat16, torch.float16):
        from flash_attn import flash_attn_varlen_func
        mq = max(b - a for a, b in zip(cu_q[:-1], cu_q[1:]))
        mk = max(b - a for a, b in zip(cu_k[:-1], cu_k[1:]))
        ws = (-1, -1) if window is None else (int(window[0]), 0)
        vpad = vv if vv.shape[-1] == qq.shape[-1] else torch.nn.functional.pad(vv, (0, qq.shape[-1] - vv.shape[-1]))
        o = flash_attn_varlen_func(qq, kk, vpad, cuq, cuk, mq, mk, softmax_scale=scale, causal=True, window_size=ws)
        o = o[..., :vv.shape[-1]]
    else:
        o = attention_ref(qq, kk, vv, cuq, cuk, True, scale, window, sinks)
    # entries were appended in local order, so the output already is in local token order
    return o
