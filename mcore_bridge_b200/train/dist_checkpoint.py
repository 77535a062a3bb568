"""Layout-independent sharded checkpoints of the model (and adapter) parameters.

Every parameter is described by where its local shard sits in the *global* tensor (``sharded_state_dict``): the key
with the global layer index, the global shape, the offset of this rank's piece along each dim, and whether this rank
is the one that writes it (replicas are written once).  The description is derived from the sharding attributes the
layers put on their parameters (``tensor_model_parallel`` / ``partition_dim`` / ``partition_stride`` for tensor
parallelism, ``is_expert`` plus a leading expert dim for expert parallelism) and from the pipeline stage's layer
offset, so every module takes part without code of its own.  ``save`` writes one safetensors file per rank plus a
manifest of all pieces; ``load`` fills each local shard from whatever saved pieces overlap it, so a checkpoint written
under one TP / PP / EP layout loads under any other.

Parity: the reference's modules take part in Megatron's distributed checkpointing through ``sharded_state_dict``
overrides (``src/mcore_bridge/model/gpt_model.py:584-621``,
``src/mcore_bridge/model/modules/gated_delta_net.py:381-425``,
``src/mcore_bridge/tuners/lora.py:448-474``, ``src/mcore_bridge/tuners/utils.py:8-28``); this module is that
checkpoint format's counterpart here.  (Model exchange with Transformers stays on the Hugging Face bridge; the
optimizer state has its own per-rank format in ``train/checkpoint.py``.)
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch
import torch.distributed as dist
from safetensors import safe_open
from safetensors.torch import save_file

from ..parallel import state as ps


@dataclass
class ShardedTensor:
    key: str                       # global name (pipeline-independent layer index)
    data: torch.Tensor             # this rank's piece (a view of the parameter)
    global_shape: Tuple[int, ...]
    global_offset: Tuple[int, ...]
    writer: bool                   # this rank writes the piece (exactly one rank per distinct piece does)


def _rank_in(name: str) -> int:
    return ps.get_rank_in(name) if ps.get_world_size(name) > 1 else 0


def _global_name(name: str, layer_offset: int) -> str:
    m = re.match(r'(.*decoder\.layers\.)(\d+)(\..*)', name)
    if m is None:
        return name
    return f'{m.group(1)}{int(m.group(2)) + layer_offset}{m.group(3)}'


def sharded_state_dict(models: Iterable[torch.nn.Module], prefix: str = '', trainable_only: bool = False
                       ) -> Dict[str, List[ShardedTensor]]:
    """``{key: pieces}`` for every parameter and persistent buffer of the model chunks this rank holds.  A parameter
    whose local shard interleaves several partitions (the ``[gate; up]`` stacking of gated MLPs) yields one piece per
    partition."""
    from ..utils.megatron_utils import unwrap_model
    out: Dict[str, List[ShardedTensor]] = {}
    dp0 = _rank_in('dp') == 0 and _rank_in('cp') == 0
    edp0 = _rank_in('edp') == 0
    for model in unwrap_model(list(models)):
        inner = model
        while hasattr(inner, 'base_model') or (hasattr(inner, 'model') and not hasattr(inner, 'decoder')):
            inner = inner.base_model if hasattr(inner, 'base_model') else inner.model
        lm = getattr(inner, 'language_model', inner)
        offset = lm.decoder.layer_offset if hasattr(lm, 'decoder') else 0
        named = list(model.named_parameters()) + [(n, b) for n, b in model.named_buffers()
                                                  if n.rsplit('.', 1)[-1] not in
                                                  model.get_submodule(n.rsplit('.', 1)[0] if '.' in n else '')
                                                  ._non_persistent_buffers_set]
        for name, p in named:
            if trainable_only and not getattr(p, 'requires_grad', False):
                continue
            is_expert = bool(getattr(p, 'is_expert', False))
            tp_name = 'etp' if is_expert else 'tp'
            tp, tp_rank = ps.get_world_size(tp_name), _rank_in(tp_name)
            sharded = bool(getattr(p, 'tensor_model_parallel', False)) and tp > 1
            pdim = int(getattr(p, 'partition_dim', -1))
            stride = int(getattr(p, 'partition_stride', 1) or 1)
            shape = list(p.shape)
            gshape, goff = list(shape), [0] * len(shape)
            if sharded:
                gshape[pdim] = shape[pdim] * tp
                goff[pdim] = shape[pdim] * tp_rank
            ep = ps.get_world_size('ep')
            stacked = is_expert and p.dim() >= 2 and ep > 1 and 'experts' in name
            if stacked:
                gshape[0] = shape[0] * ep
                goff[0] = shape[0] * _rank_in('ep')
            writer = (edp0 if is_expert else dp0) and (sharded or tp_rank == 0)
            if getattr(p, 'shared_embedding', False) and not ps.is_pipeline_first_stage():
                writer = False          # a tied embedding lives on both pipeline ends: the first stage writes it
            key = prefix + _global_name(name, offset)
            data = p.detach()
            if sharded and stride > 1 and shape[pdim] % stride == 0:
                # local [s0; s1; ...] along pdim, each a shard of its own partition of the global tensor
                pieces = []
                loc = shape[pdim] // stride
                for j in range(stride):
                    off = list(goff)
                    off[pdim] = j * (gshape[pdim] // stride) + loc * tp_rank
                    pieces.append(ShardedTensor(key, data.narrow(pdim, j * loc, loc), tuple(gshape), tuple(off),
                                                writer))
                out[key] = pieces
            else:
                out[key] = [ShardedTensor(key, data, tuple(gshape), tuple(goff), writer)]
    return out


def save(models, directory: str, prefix: str = '', trainable_only: bool = False) -> None:
    """Collective over all ranks: every rank writes the pieces it is the writer of, rank 0 writes the manifest."""
    os.makedirs(directory, exist_ok=True)
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    fname = f'shard_{rank:05d}.safetensors'
    tensors, entries = {}, []
    for key, pieces in sharded_state_dict(models, prefix, trainable_only).items():
        for j, st in enumerate(pieces):
            if not st.writer:
                continue
            name = f'{key}#{len(tensors)}'
            tensors[name] = st.data.contiguous().cpu()
            entries.append({'key': key, 'file': fname, 'name': name, 'global_shape': list(st.global_shape),
                            'offset': list(st.global_offset), 'shape': list(st.data.shape),
                            'dtype': str(st.data.dtype).replace('torch.', '')})
    if tensors:
        save_file(tensors, os.path.join(directory, fname))
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, entries)
    else:
        gathered = [entries]
    if rank == 0:
        manifest: Dict[str, list] = {}
        for part in gathered:
            for e in part:
                manifest.setdefault(e['key'], []).append(e)
        with open(os.path.join(directory, 'manifest.json'), 'w', encoding='utf-8') as f:
            json.dump({'format': 'mcore_bridge_b200.dist_checkpoint/1', 'tensors': manifest}, f)
    if world > 1:
        dist.barrier()


def _overlap(a_off, a_shape, b_off, b_shape):
    """Intersection of two boxes: (slices into a, slices into b) or None."""
    sa, sb = [], []
    for ao, an, bo, bn in zip(a_off, a_shape, b_off, b_shape):
        lo, hi = max(ao, bo), min(ao + an, bo + bn)
        if lo >= hi:
            return None
        sa.append(slice(lo - ao, hi - ao))
        sb.append(slice(lo - bo, hi - bo))
    return tuple(sa), tuple(sb)


def load(models, directory: str, prefix: str = '', strict: bool = True, trainable_only: bool = False) -> List[str]:
    """Fills every local shard from the saved pieces that overlap it (any saving layout).  Returns the keys that were
    missing from the checkpoint (raises for them when ``strict``)."""
    with open(os.path.join(directory, 'manifest.json'), 'r', encoding='utf-8') as f:
        manifest = json.load(f)['tensors']
    handles = {}

    def handle(fn):
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(directory, fn), framework='pt', device='cpu')
        return handles[fn]

    missing = []
    with torch.no_grad():
        for key, pieces in sharded_state_dict(models, prefix, trainable_only).items():
            saved = manifest.get(key)
            if saved is None:
                missing.append(key)
                continue
            for st in pieces:
                filled = 0
                for e in saved:
                    if tuple(e['global_shape']) != st.global_shape:
                        raise ValueError(f'{key}: global shape {tuple(e["global_shape"])} in the checkpoint, '
                                         f'{st.global_shape} in the model')
                    ov = _overlap(st.global_offset, st.data.shape, e['offset'], e['shape'])
                    if ov is None:
                        continue
                    src = handle(e['file']).get_tensor(e['name'])
                    st.data[ov[0]].copy_(src[ov[1]].to(device=st.data.device, dtype=st.data.dtype))
                    n = 1
                    for s in ov[0]:
                        n *= s.stop - s.start
                    filled += n
                if filled < st.data.numel():
                    raise ValueError(f'{key}: the checkpoint covers only {filled} of {st.data.numel()} elements of the '
                                     f'local shard at offset {st.global_offset}')
    if missing and strict:
        raise KeyError(f'missing from the checkpoint: {missing[:8]}{" ..." if len(missing) > 8 else ""}')
    return missing
