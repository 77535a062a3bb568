"""Differentiable collectives over the tensor / context / expert groups (library path).

These are the ``torch.distributed`` implementations: the CPU/gloo test path, the baseline the fused
sm_100a kernels are compared against, and the fallback for shapes the fused kernels do not take.
Activations are token-major ``[T, ...]``; sequence parallelism shards dim 0.

Parity: the gather/scatter/reduce call sites listed for the reference in
``src/mcore_bridge/model/modules/transformer_layer.py:350-374`` and ``model/gpt_model.py:400-412``.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import state as ps


def _size(group_name: str) -> int:
    return ps.get_world_size(group_name)


def all_reduce(x: torch.Tensor, group_name: str = 'tp', op=dist.ReduceOp.SUM) -> torch.Tensor:
    if _size(group_name) == 1:
        return x
    dist.all_reduce(x, op=op, group=ps.get_group(group_name))
    return x


def all_gather_dim0(x: torch.Tensor, group_name: str = 'tp') -> torch.Tensor:
    n = _size(group_name)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] * n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=ps.get_group(group_name))
    return out


def reduce_scatter_dim0(x: torch.Tensor, group_name: str = 'tp') -> torch.Tensor:
    n = _size(group_name)
    if n == 1:
        return x
    x = x.contiguous()
    assert x.shape[0] % n == 0, f'dim 0 ({x.shape[0]}) not divisible by group size {n}'
    out = torch.empty((x.shape[0] // n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.device.type == 'cpu':
        # gloo has no reduce_scatter_tensor: all-reduce then slice
        tmp = x.clone()
        dist.all_reduce(tmp, group=ps.get_group(group_name))
        r = ps.get_rank_in(group_name)
        out.copy_(tmp[r * out.shape[0]:(r + 1) * out.shape[0]])
    else:
        dist.reduce_scatter_tensor(out, x, group=ps.get_group(group_name))
    return out


def split_dim0(x: torch.Tensor, group_name: str = 'tp') -> torch.Tensor:
    n = _size(group_name)
    if n == 1:
        return x
    r = ps.get_rank_in(group_name)
    assert x.shape[0] % n == 0
    c = x.shape[0] // n
    return x[r * c:(r + 1) * c].contiguous()


def all_gather_last_dim(x: torch.Tensor, group_name: str = 'tp') -> torch.Tensor:
    n = _size(group_name)
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=ps.get_group(group_name))
    return torch.cat(parts, dim=-1)


def split_last_dim(x: torch.Tensor, group_name: str = 'tp') -> torch.Tensor:
    n = _size(group_name)
    if n == 1:
        return x
    r = ps.get_rank_in(group_name)
    c = x.shape[-1] // n
    return x[..., r * c:(r + 1) * c].contiguous()


class _CopyToRegion(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel linear without SP)."""

    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce(g.contiguous().clone(), ctx.group_name), None


class _ReduceFromRegion(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel linear without SP)."""

    @staticmethod
    def forward(ctx, x, group_name):
        return all_reduce(x.contiguous().clone(), group_name)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterToSequenceRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        return split_dim0(x, group_name)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group_name), None


class _GatherFromSequenceRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group_name, reduce_scatter_grad):
        ctx.group_name, ctx.rs = group_name, reduce_scatter_grad
        return all_gather_dim0(x, group_name)

    @staticmethod
    def backward(ctx, g):
        if ctx.rs:
            return reduce_scatter_dim0(g, ctx.group_name), None, None
        return split_dim0(g, ctx.group_name), None, None


class _ReduceScatterToSequenceRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        return reduce_scatter_dim0(x, group_name)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group_name), None


class _GatherLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        return all_gather_last_dim(x, group_name)

    @staticmethod
    def backward(ctx, g):
        return split_last_dim(g, ctx.group_name), None


class _ScatterLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        return split_last_dim(x, group_name)

    @staticmethod
    def backward(ctx, g):
        return all_gather_last_dim(g, ctx.group_name), None


class _GatherLastDimSum(torch.autograd.Function):
    """All-gather on the last dim whose consumers differ per rank: the gradients of the gathered tensor are summed over
    the group and each rank keeps the slice it produced (reduce-scatter on the last dim)."""

    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        return all_gather_last_dim(x, group_name)

    @staticmethod
    def backward(ctx, g):
        return split_last_dim(all_reduce(g.contiguous().clone(), ctx.group_name), ctx.group_name), None


def all_gather_last_dim_sum_grad(x, group_name: str = 'tp'):
    return x if _size(group_name) == 1 else _GatherLastDimSum.apply(x, group_name)


class _AllReduceBoth(torch.autograd.Function):
    """Sum over the group in forward *and* backward: for statistics shared by ranks whose downstream computation
    differs (each rank's loss term depends on every rank's contribution to the statistic)."""

    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        return all_reduce(x.clone(), group_name)

    @staticmethod
    def backward(ctx, g):
        return all_reduce(g.clone(), ctx.group_name), None


def all_reduce_both(x, group_name: str = 'tp'):
    if _size(group_name) == 1:
        return x
    return _AllReduceBoth.apply(x, group_name)


def copy_to_tensor_model_parallel_region(x, group_name: str = 'tp'):
    return x if _size(group_name) == 1 else _CopyToRegion.apply(x, group_name)


def reduce_from_tensor_model_parallel_region(x, group_name: str = 'tp'):
    return x if _size(group_name) == 1 else _ReduceFromRegion.apply(x, group_name)


def scatter_to_sequence_parallel_region(x, group_name: str = 'tp'):
    return x if _size(group_name) == 1 else _ScatterToSequenceRegion.apply(x, group_name)


def gather_from_sequence_parallel_region(x, group_name: str = 'tp', tensor_parallel_output_grad: bool = True):
    """All-gather on dim 0.  ``tensor_parallel_output_grad``: the consumer is tensor-parallel, so the
    gradients differ per rank and are reduce-scattered; otherwise they are identical and simply split."""
    return x if _size(group_name) == 1 else _GatherFromSequenceRegion.apply(x, group_name, tensor_parallel_output_grad)


def reduce_scatter_to_sequence_parallel_region(x, group_name: str = 'tp'):
    return x if _size(group_name) == 1 else _ReduceScatterToSequenceRegion.apply(x, group_name)


def gather_from_tensor_model_parallel_region(x, group_name: str = 'tp'):
    return x if _size(group_name) == 1 else _GatherLastDim.apply(x, group_name)


def scatter_to_tensor_model_parallel_region(x, group_name: str = 'tp'):
    return x if _size(group_name) == 1 else _ScatterLastDim.apply(x, group_name)


# ------------------------------------------------------------------ all-to-all
def all_to_all_single(x: torch.Tensor, out_splits: Optional[List[int]], in_splits: Optional[List[int]],
                      group_name: str) -> torch.Tensor:
    n = _size(group_name)
    if n == 1:
        return x
    x = x.contiguous()
    group = ps.get_group(group_name)
    if out_splits is None:
        out = torch.empty_like(x)
    else:
        out = torch.empty((sum(out_splits), *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.device.type == 'cpu':
        # gloo: emulate with all_gather of padded chunks
        ins = list(x.split(in_splits if in_splits is not None else x.shape[0] // n, dim=0))
        outs = [None] * n
        r = ps.get_rank_in(group_name)
        gathered = [None] * n
        dist.all_gather_object(gathered, [t.clone() for t in ins], group=group)
        for src in range(n):
            outs[src] = gathered[src][r]
        return torch.cat(outs, dim=0)
    dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    return out


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group_name):
        ctx.out_splits, ctx.in_splits, ctx.group_name = out_splits, in_splits, group_name
        return all_to_all_single(x, out_splits, in_splits, group_name)

    @staticmethod
    def backward(ctx, g):
        return all_to_all_single(g, ctx.in_splits, ctx.out_splits, ctx.group_name), None, None, None


def all_to_all(x, out_splits=None, in_splits=None, group_name: str = 'ep'):
    return x if _size(group_name) == 1 else _AllToAll.apply(x, out_splits, in_splits, group_name)


def all_to_all_cp2hp(x: torch.Tensor, group_name: str = 'cp') -> torch.Tensor:
    """``[T/cp, D] -> [T, D/cp]``: sequence-sharded to head-sharded (gated-DeltaNet under CP).

    Parity: reference ``src/mcore_bridge/model/modules/gated_delta_net.py:206-227``.
    """
    n = _size(group_name)
    if n == 1:
        return x
    t, d = x.shape[0], x.shape[-1]
    assert d % n == 0
    xs = x.reshape(t, n, d // n).transpose(0, 1).contiguous().reshape(n * t, d // n)  # chunk j -> rank j
    return all_to_all(xs, None, None, group_name)  # result rows: [src rank, t]


def all_to_all_hp2cp(x: torch.Tensor, group_name: str = 'cp') -> torch.Tensor:
    """``[T, D/cp] -> [T/cp, D]``: inverse of :func:`all_to_all_cp2hp`."""
    n = _size(group_name)
    if n == 1:
        return x
    T, dl = x.shape
    t = T // n
    y = all_to_all(x.contiguous(), None, None, group_name)  # rows: [src rank j, t] holding head slice j
    return y.reshape(n, t, dl).transpose(0, 1).reshape(t, n * dl)
