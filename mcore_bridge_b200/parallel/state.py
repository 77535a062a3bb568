"""Process-group mesh: TP / CP / DP / PP for dense parameters and ETP / EP / EDP / PP for experts.

One process per GPU.  Rank order is ``tp-cp-ep-dp-pp`` (tensor parallel fastest), the order the
reference's bridge assumes when it derives its own groups (reference
``src/mcore_bridge/bridge/gpt_bridge.py:73-113``).  Dense view: ``world = tp * cp * dp * pp``;
expert view of the same ranks: ``world = etp * ep * edp * pp``.

Backend: ``nccl`` on GPUs, ``gloo`` on CPU (tests).  With ``world_size == 1`` and no initialised
``torch.distributed`` every query answers as a single-rank mesh, so models run without a launcher.
"""
from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

_STATE: Optional['ParallelState'] = None


def _decompose(rank: int, sizes: Sequence[int]) -> List[int]:
    out = []
    for s in sizes:
        out.append(rank % s)
        rank //= s
    return out


def _compose(coords: Sequence[int], sizes: Sequence[int]) -> int:
    rank, mul = 0, 1
    for c, s in zip(coords, sizes):
        rank += c * mul
        mul *= s
    return rank


def groups_for(world: int, names: Sequence[str], sizes: Sequence[int], token: Sequence[str]) -> List[List[int]]:
    """All rank lists that vary over the axes in ``token`` (in axis order) with the other axes fixed."""
    assert world == int(torch.tensor(sizes).prod()), (world, sizes)
    vary = [i for i, n in enumerate(names) if n in token]
    fixed = [i for i in range(len(names)) if i not in vary]
    out = []
    for fixed_coords in itertools.product(*[range(sizes[i]) for i in reversed(fixed)]):
        fixed_coords = list(reversed(fixed_coords))
        ranks = []
        for vary_coords in itertools.product(*[range(sizes[i]) for i in reversed(vary)]):
            vary_coords = list(reversed(vary_coords))
            coords = [0] * len(names)
            for i, c in zip(fixed, fixed_coords):
                coords[i] = c
            for i, c in zip(vary, vary_coords):
                coords[i] = c
            ranks.append(_compose(coords, sizes))
        out.append(ranks)
    return out


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    tp: int = 1
    cp: int = 1
    dp: int = 1
    pp: int = 1
    vpp: Optional[int] = None
    ep: int = 1
    etp: int = 1
    edp: int = 1
    groups: Dict[str, Optional[dist.ProcessGroup]] = field(default_factory=dict)
    group_ranks: Dict[str, List[int]] = field(default_factory=dict)
    vp_rank: Optional[int] = None

    # dense axes, fastest first
    @property
    def dense_names(self):
        return ('tp', 'cp', 'dp', 'pp')

    @property
    def dense_sizes(self):
        return (self.tp, self.cp, self.dp, self.pp)

    @property
    def expert_names(self):
        return ('etp', 'ep', 'edp', 'pp')

    @property
    def expert_sizes(self):
        return (self.etp, self.ep, self.edp, self.pp)

    def coords(self) -> Dict[str, int]:
        d = dict(zip(self.dense_names, _decompose(self.rank, self.dense_sizes)))
        d.update(zip(self.expert_names, _decompose(self.rank, self.expert_sizes)))
        return d


# name -> (view, axes)
_GROUP_DEFS = {
    'tp': ('dense', ('tp',)),
    'cp': ('dense', ('cp',)),
    'dp': ('dense', ('dp',)),
    'dp_cp': ('dense', ('cp', 'dp')),
    'tp_cp': ('dense', ('tp', 'cp')),
    'tp_dp_cp': ('dense', ('tp', 'cp', 'dp')),
    'pp': ('dense', ('pp',)),
    'pp_bwd': ('dense', ('pp',)),     # second communicator over the same ranks: gradients travel on it, so a rank
                                      # pair's activation and gradient messages never share an ordered channel
    'mp': ('dense', ('tp', 'pp')),
    'etp': ('expert', ('etp',)),
    'ep': ('expert', ('ep',)),
    'edp': ('expert', ('edp',)),
    'etp_ep': ('expert', ('etp', 'ep')),
    'ep_pp': ('expert', ('ep', 'pp')),
}


def initialize_model_parallel(tensor_model_parallel_size: int = 1, pipeline_model_parallel_size: int = 1,
                              virtual_pipeline_model_parallel_size: Optional[int] = None,
                              context_parallel_size: int = 1, expert_model_parallel_size: int = 1,
                              expert_tensor_parallel_size: Optional[int] = None,
                              backend: Optional[str] = None, timeout_s: Optional[float] = None) -> ParallelState:
    """Builds every process group.  ``torch.distributed`` must be initialised unless world size is 1."""
    global _STATE
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()
    else:
        world, rank = 1, 0
    tp, pp, cp, ep = (tensor_model_parallel_size, pipeline_model_parallel_size, context_parallel_size,
                      expert_model_parallel_size)
    etp = tp if expert_tensor_parallel_size is None else expert_tensor_parallel_size
    if world % (tp * cp * pp) != 0:
        raise ValueError(f'world size {world} is not divisible by tp*cp*pp = {tp * cp * pp}')
    dp = world // (tp * cp * pp)
    if world % (etp * ep * pp) != 0:
        raise ValueError(f'world size {world} is not divisible by etp*ep*pp = {etp * ep * pp}')
    edp = world // (etp * ep * pp)
    st = ParallelState(world_size=world, rank=rank, tp=tp, cp=cp, dp=dp, pp=pp,
                       vpp=virtual_pipeline_model_parallel_size, ep=ep, etp=etp, edp=edp)
    if virtual_pipeline_model_parallel_size is not None:
        st.vp_rank = 0
    kw = {}
    if timeout_s is not None:
        kw['timeout'] = timedelta(seconds=timeout_s)
    for name, (view, axes) in _GROUP_DEFS.items():
        names, sizes = (st.dense_names, st.dense_sizes) if view == 'dense' else (st.expert_names, st.expert_sizes)
        mine, handle = None, None
        for ranks in groups_for(world, names, sizes, axes):
            if world > 1:
                g = dist.new_group(ranks, backend=backend, **kw) if len(ranks) > 1 else None
            else:
                g = None
            if rank in ranks:
                mine, handle = ranks, g
        st.group_ranks[name] = mine
        st.groups[name] = handle
    # embedding group: first and last pipeline stage of every pipeline (tied input / output embeddings keep one
    # copy on each and sum their gradients); ranks in between are not members
    mine, handle = None, None
    for ranks in groups_for(world, st.dense_names, st.dense_sizes, ('pp',)):
        ends = [ranks[0], ranks[-1]] if len(ranks) > 1 else [ranks[0]]
        g = dist.new_group(ends, backend=backend, **kw) if (world > 1 and len(ends) > 1) else None
        if rank in ends:
            mine, handle = ends, g
    st.group_ranks['embd'] = mine
    st.groups['embd'] = handle
    _STATE = st
    return st


def destroy_model_parallel():
    global _STATE
    _STATE = None


def model_parallel_is_initialized() -> bool:
    return _STATE is not None


def get_state() -> ParallelState:
    global _STATE
    if _STATE is None:
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            raise RuntimeError('call initialize_model_parallel() first')
        _STATE = ParallelState()
        for name in list(_GROUP_DEFS) + ['embd']:
            _STATE.groups[name] = None
            _STATE.group_ranks[name] = [0]
    return _STATE


def get_group(name: str):
    return get_state().groups.get(name)


def get_group_ranks(name: str) -> List[int]:
    return get_state().group_ranks[name]


def get_world_size(name: str) -> int:
    return len(get_state().group_ranks[name])


def get_rank_in(name: str) -> int:
    st = get_state()
    return st.group_ranks[name].index(st.rank)


# ---- Megatron-style accessors (the names user scripts written for the reference expect)
def get_tensor_model_parallel_group():
    return get_group('tp')


def get_tensor_model_parallel_world_size() -> int:
    return get_state().tp


def get_tensor_model_parallel_rank() -> int:
    return get_state().coords()['tp']


def get_context_parallel_group():
    return get_group('cp')


def get_context_parallel_world_size() -> int:
    return get_state().cp


def get_context_parallel_rank() -> int:
    return get_state().coords()['cp']


def get_pipeline_model_parallel_group():
    return get_group('pp')


def get_pipeline_model_parallel_world_size() -> int:
    return get_state().pp


def get_pipeline_model_parallel_rank() -> int:
    return get_state().coords()['pp']


def get_virtual_pipeline_model_parallel_world_size() -> Optional[int]:
    return get_state().vpp


def get_virtual_pipeline_model_parallel_rank() -> Optional[int]:
    return get_state().vp_rank


def set_virtual_pipeline_model_parallel_rank(r: Optional[int]):
    get_state().vp_rank = r


def is_pipeline_first_stage(ignore_virtual: bool = True, vp_stage: Optional[int] = None) -> bool:
    st = get_state()
    if not ignore_virtual and st.vpp is not None and st.vpp > 1:
        if (vp_stage if vp_stage is not None else st.vp_rank) != 0:
            return False
    return st.coords()['pp'] == 0


def is_pipeline_last_stage(ignore_virtual: bool = True, vp_stage: Optional[int] = None) -> bool:
    st = get_state()
    if not ignore_virtual and st.vpp is not None and st.vpp > 1:
        if (vp_stage if vp_stage is not None else st.vp_rank) != st.vpp - 1:
            return False
    return st.coords()['pp'] == st.pp - 1


def get_pipeline_model_parallel_next_rank() -> int:
    st = get_state()
    ranks = st.group_ranks['pp']
    return ranks[(ranks.index(st.rank) + 1) % len(ranks)]


def get_pipeline_model_parallel_prev_rank() -> int:
    st = get_state()
    ranks = st.group_ranks['pp']
    return ranks[(ranks.index(st.rank) - 1) % len(ranks)]


def get_data_parallel_group(with_context_parallel: bool = False):
    return get_group('dp_cp' if with_context_parallel else 'dp')


def get_data_parallel_world_size(with_context_parallel: bool = False) -> int:
    return get_world_size('dp_cp' if with_context_parallel else 'dp')


def get_data_parallel_rank(with_context_parallel: bool = False) -> int:
    return get_rank_in('dp_cp' if with_context_parallel else 'dp')


def get_expert_model_parallel_group():
    return get_group('ep')


def get_expert_model_parallel_world_size() -> int:
    return get_state().ep


def get_expert_model_parallel_rank() -> int:
    return get_state().coords()['ep']


def get_expert_tensor_parallel_group():
    return get_group('etp')


def get_expert_tensor_parallel_world_size() -> int:
    return get_state().etp


def get_expert_tensor_parallel_rank() -> int:
    return get_state().coords()['etp']


def get_expert_data_parallel_group():
    return get_group('edp')


def get_expert_data_parallel_world_size() -> int:
    return get_state().edp


def get_expert_data_parallel_rank() -> int:
    return get_state().coords()['edp']


def get_expert_pipeline_group():
    """EP x PP group the bridge broadcasts expert weights over on export."""
    return get_group('ep_pp')


def get_model_parallel_group():
    return get_group('mp')


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0, store=None) -> None:
    """Initialises ``torch.distributed`` from the torchrun environment (no-op for a single process).  ``store``: an
    explicit rendezvous store instead of the environment's (for a second initialisation after ``exec``)."""
    if dist.is_initialized():
        return
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world <= 1 and 'RANK' not in os.environ:
        return
    if backend is None:
        backend = 'nccl' if torch.cuda.is_available() else 'gloo'
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
    kw = {}
    if backend == 'nccl':
        kw['device_id'] = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
    if store is not None:
        kw.update(store=store, rank=int(os.environ['RANK']), world_size=world)
    dist.init_process_group(backend=backend, timeout=timedelta(seconds=timeout_s), **kw)
