"""Sequence / context-parallel helpers with the reference's public names.

* :func:`split_cp_inputs` — zig-zag ``2*cp`` chunking of each (packed) sequence, this rank keeps chunks
  ``r`` and ``2cp-1-r`` (reference ``src/mcore_bridge/utils/megatron_utils.py:48-68``).
* :func:`reconstruct_tensor_cp` — inverse: all-gather over CP and undo the zig-zag (``:71-106``).
* :func:`roll_tensor` — one-token left shift that respects packed-sequence boundaries and, under CP, fetches
  the boundary tokens of neighbouring chunks with ONE all-gather (the reference exchanges them per sequence
  with isend/irecv, ``:147-242``).
* :func:`set_random_seed`, :func:`unwrap_model`, :func:`get_local_layer_specs`.
"""
from __future__ import annotations

import random
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import state as ps
from .torch_utils import host_list


def unwrap_model(models, module_instances=None):
    """Strips wrapper modules (DDP, our ``DistributedDataParallel``, half-precision wrappers, PEFT)."""
    from torch.nn.parallel import DistributedDataParallel as TorchDDP
    if module_instances is None:
        wrappers = [TorchDDP]
        try:
            from ..train.distributed_optimizer import DistributedDataParallel as OurDDP
            wrappers.append(OurDDP)
        except Exception:
            pass
        module_instances = tuple(wrappers)
    return_list = isinstance(models, (list, tuple))
    if not return_list:
        models = [models]
    out = []
    for m in models:
        while isinstance(m, module_instances):
            m = m.module
        out.append(m)
    return out if return_list else out[0]


def _cp_rank_size(cp_size=None, cp_rank=None):
    if cp_size is None:
        cp_size = ps.get_context_parallel_world_size()
    if cp_rank is None:
        cp_rank = ps.get_context_parallel_rank() if cp_size > 1 else 0
    return cp_size, cp_rank


def split_cp_inputs(inputs: torch.Tensor, cu_seqlens: Optional[torch.Tensor], dim: int,
                    cp_size: Optional[int] = None, cp_rank: Optional[int] = None) -> torch.Tensor:
    """Keeps this CP rank's two zig-zag chunks of every sequence along ``dim``.

    ``cu_seqlens`` delimits packed sequences along ``dim`` (each length a multiple of ``2*cp``); ``None``
    treats the whole dimension as one sequence.
    """
    cp_size, cp_rank = _cp_rank_size(cp_size, cp_rank)
    if cp_size == 1:
        return inputs
    if dim < 0:
        dim += inputs.ndim
    bounds = [0, inputs.shape[dim]] if cu_seqlens is None else host_list(cu_seqlens)
    idx = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        n = e - s
        assert n % (2 * cp_size) == 0, f'sequence length {n} not divisible by 2*cp = {2 * cp_size}'
        c = n // (2 * cp_size)
        idx.append(torch.arange(s + cp_rank * c, s + (cp_rank + 1) * c))
        idx.append(torch.arange(s + (2 * cp_size - cp_rank - 1) * c, s + (2 * cp_size - cp_rank) * c))
    index = torch.cat(idx).to(inputs.device)
    return inputs.index_select(dim, index)


def cp_gather_index(cu_seqlens: Optional[torch.Tensor], total: int, cp_size: int) -> torch.Tensor:
    """``index[j]`` = position in the rank-major concatenation ``[rank0 tokens | rank1 tokens | ...]`` of the
    ``j``-th token of the original stream (used to undo the zig-zag after an all-gather)."""
    bounds = [0, total] if cu_seqlens is None else host_list(cu_seqlens)
    local_total = total // cp_size
    out = torch.empty(total, dtype=torch.int64)
    local_off = 0
    for s, e in zip(bounds[:-1], bounds[1:]):
        n = e - s
        c = n // (2 * cp_size)
        for r in range(cp_size):
            base = r * local_total + local_off
            out[s + r * c:s + (r + 1) * c] = torch.arange(base, base + c)
            out[s + (2 * cp_size - r - 1) * c:s + (2 * cp_size - r) * c] = torch.arange(base + c, base + 2 * c)
        local_off += 2 * c
    return out


def reconstruct_tensor_cp(tensor: torch.Tensor, packed_seq_params=None, dim: int = 1) -> torch.Tensor:
    """All-gathers a CP-sharded tensor along ``dim`` and restores the original token order."""
    cp_size = ps.get_context_parallel_world_size()
    if cp_size <= 1:
        return tensor
    group = ps.get_context_parallel_group()
    parts = [torch.empty_like(tensor) for _ in range(cp_size)]
    dist.all_gather(parts, tensor.contiguous(), group=group)
    parts[ps.get_context_parallel_rank()] = tensor  # keep autograd for the local part
    gathered = torch.cat(parts, dim=dim)
    cu = None if packed_seq_params is None else packed_seq_params.cu_seqlens_q
    index = cp_gather_index(cu, gathered.shape[dim], cp_size).to(tensor.device)
    return gathered.index_select(dim, index)


def get_local_layer_specs(config, layer_specs: List, vp_stage: Optional[int] = None) -> List:
    """The slice of a per-layer list owned by this pipeline (virtual) stage."""
    from ..models.transformer_block import get_num_layers_to_build, get_transformer_layer_offset
    n = get_num_layers_to_build(config, vp_stage)
    off = get_transformer_layer_offset(config, vp_stage)
    return layer_specs[off:off + n]


def set_random_seed(seed_: int, data_parallel_random_init: bool = False, te_rng_tracker: bool = False,
                    inference_rng_tracker: bool = False, use_cudagraphable_rng: bool = False) -> None:
    """Seeds python / numpy / torch: ``seed + 1009 * pp_rank (+ 11 * dp_rank)`` and the tensor-parallel RNG
    tracker (reference ``src/mcore_bridge/utils/megatron_utils.py:124-143``)."""
    if seed_ is None or seed_ <= 0:
        raise ValueError(f'Seed ({seed_}) should be a positive integer.')
    seed = seed_ + 1009 * ps.get_pipeline_model_parallel_rank()
    if data_parallel_random_init:
        seed += 11 * ps.get_data_parallel_rank()
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    from ..parallel.random import model_parallel_manual_seed
    model_parallel_manual_seed(seed)


def _roll_packed(tensor: torch.Tensor, cu: torch.Tensor) -> torch.Tensor:
    T = tensor.shape[-1]
    rolled = torch.roll(tensor, shifts=-1, dims=-1)
    last = (cu[1:].to(torch.int64) - 1).to(tensor.device)
    last = last[(last >= 0) & (last < T)]
    mask = torch.zeros(T, dtype=torch.bool, device=tensor.device)
    mask[last] = True
    mask[T - 1] = True
    return rolled.masked_fill(mask, 0)


def roll_tensor(tensor: torch.Tensor, shifts: int = -1, dims: int = -1, cp_group=None, packed_seq_params=None):
    """Left-shift by one token along the last dim; positions whose successor lies in another sequence (or past
    the end) become 0.  Returns ``(rolled, rolled.sum())`` like the reference."""
    assert shifts == -1 and (dims == -1 or dims == tensor.dim() - 1), 'only a one-token left shift is supported'
    cp_size = 1 if cp_group is None else dist.get_world_size(cp_group)
    cu = None if packed_seq_params is None else packed_seq_params.cu_seqlens_q
    T = tensor.shape[-1]
    if cp_size == 1:
        if cu is None:
            rolled = torch.roll(tensor, -1, -1)
            rolled[..., -1] = 0
        else:
            rolled = _roll_packed(tensor, cu)
        return rolled, rolled.sum()
    rank = dist.get_rank(cp_group)
    # local layout per sequence: [front chunk r | tail chunk 2cp-1-r], each of length c_i
    bounds = [0, T * cp_size] if cu is None else host_list(cu)
    starts, lens = [], []
    off = 0
    for s, e in zip(bounds[:-1], bounds[1:]):
        c = (e - s) // (2 * cp_size)
        starts.append(off)
        lens.append(c)
        off += 2 * c
    dev = tensor.device
    st = torch.tensor(starts, device=dev)
    ln = torch.tensor(lens, device=dev)
    nz = ln > 0
    first_front = tensor.index_select(-1, torch.where(nz, st, torch.zeros_like(st)))         # [..., S]
    first_tail = tensor.index_select(-1, torch.where(nz, st + ln, torch.zeros_like(st)))
    mine = torch.stack((first_front, first_tail), dim=-1).contiguous()                         # [..., S, 2]
    allb = [torch.empty_like(mine) for _ in range(cp_size)]
    dist.all_gather(allb, mine, group=cp_group)
    rolled = torch.roll(tensor, -1, -1)
    # successor of the front chunk: front of rank+1, or own tail on the last rank
    nxt_front = allb[rank + 1][..., 0] if rank < cp_size - 1 else first_tail
    # successor of the tail chunk: tail of rank-1, or nothing on rank 0
    nxt_tail = allb[rank - 1][..., 1] if rank > 0 else torch.zeros_like(first_tail)
    idx_front_last = (st + ln - 1)[nz]
    idx_tail_last = (st + 2 * ln - 1)[nz]
    rolled[..., idx_front_last] = nxt_front[..., nz]
    rolled[..., idx_tail_last] = nxt_tail[..., nz]
    return rolled, rolled.sum()
