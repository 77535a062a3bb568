"""Training-state checkpoint / resume: optimizer shards, step, RNG streams, data position.

Model weights travel as Hugging Face safetensors through the bridge (``GPTBridge.save_weights`` /
``load_weights``).  What the bridge does not carry is saved here, one safetensors file per rank plus a JSON
manifest written by rank 0 with the parallel layout, so a resume on a different layout is refused instead of
silently mis-loading (the reference keeps no optimizer / RNG / iteration state at all).

Layout of ``<dir>/``: ``manifest.json``, ``optim_rank{r:05d}.safetensors``, ``rng_rank{r:05d}.pt``.
A checkpoint is complete only when ``manifest.json`` exists (it is written last, after a barrier).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist
from safetensors.torch import load_file, save_file

from ..parallel import state as ps
from ..parallel.random import get_rng_tracker


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _layout() -> Dict[str, int]:
    st = ps.get_state()
    return {'world_size': st.world_size, 'tp': st.tp, 'cp': st.cp, 'dp': st.dp, 'pp': st.pp, 'ep': st.ep,
            'etp': st.etp}


def _digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, 'rb') as f:
        for chunk in iter(lambda: f.read(1 << 20), b''):
            h.update(chunk)
    return h.hexdigest()


def save_training_state(trainer, directory: str, step: int, extra: Optional[dict] = None) -> None:
    os.makedirs(directory, exist_ok=True)
    r = _rank()
    sd = trainer.optimizer.state_dict()
    tensors = {}
    for i, s in enumerate(sd['shards']):
        for k, v in s.items():
            tensors[f'shard{i}.{k}'] = v.detach().cpu().contiguous()
    opath = os.path.join(directory, f'optim_rank{r:05d}.safetensors')
    save_file(tensors, opath, metadata={'step': str(sd['step'])})
    rng = {'torch': torch.get_rng_state(), 'tracker': {k: v for k, v in get_rng_tracker().states.items()}}
    if torch.cuda.is_available():
        rng['cuda'] = torch.cuda.get_rng_state()
    torch.save(rng, os.path.join(directory, f'rng_rank{r:05d}.pt'))
    digests = [None] * (dist.get_world_size() if dist.is_initialized() else 1)
    if dist.is_initialized():
        dist.all_gather_object(digests, _digest(opath))
    else:
        digests[0] = _digest(opath)
    if r == 0:
        manifest = {'step': int(step), 'optimizer_step': int(sd['step']), 'layout': _layout(), 'hyper': {
            'lr': sd['hyper']['lr'], 'betas': list(sd['hyper']['betas']), 'eps': sd['hyper']['eps'],
            'weight_decay': sd['hyper']['weight_decay']}, 'optim_sha256': digests, 'extra': extra or {}}
        tmp = os.path.join(directory, 'manifest.json.tmp')
        with open(tmp, 'w') as f:
            json.dump(manifest, f, indent=2)
        os.replace(tmp, os.path.join(directory, 'manifest.json'))
    if dist.is_initialized():
        dist.barrier()


def load_training_state(trainer, directory: str, verify: bool = True) -> dict:
    """Restores optimizer shards and RNG; returns the manifest.  Raises on a missing / corrupt / foreign checkpoint."""
    mpath = os.path.join(directory, 'manifest.json')
    if not os.path.exists(mpath):
        raise FileNotFoundError(f'{directory} holds no complete checkpoint (manifest.json missing)')
    manifest = json.load(open(mpath))
    if manifest['layout'] != _layout():
        raise ValueError(f'checkpoint layout {manifest["layout"]} differs from the running layout {_layout()}')
    r = _rank()
    opath = os.path.join(directory, f'optim_rank{r:05d}.safetensors')
    if verify and manifest.get('optim_sha256') and manifest['optim_sha256'][r] != _digest(opath):
        raise IOError(f'{opath} does not match the digest recorded in the manifest (corrupt or partial write)')
    tensors = load_file(opath)
    n = len(trainer.optimizer.shards)
    shards = []
    for i in range(n):
        shards.append({k: tensors[f'shard{i}.{k}'] for k in ('main', 'exp_avg', 'exp_avg_sq')})
    trainer.optimizer.load_state_dict({'step': manifest['optimizer_step'], 'shards': shards})
    # the bf16 parameters follow the restored master weights
    for (buf, b, _, main, _, _) in trainer.optimizer.shards:
        s, e = buf.shard_range(b)
        buf.param_data[s:e].copy_(main.to(buf.param_data.dtype))
        if buf.dp > 1:
            dist.all_gather_into_tensor(buf.param_data[b.start:b.end], buf.param_data[s:e].clone(), group=buf.group)
    rng = torch.load(os.path.join(directory, f'rng_rank{r:05d}.pt'), weights_only=False)
    torch.set_rng_state(rng['torch'])
    if 'cuda' in rng and torch.cuda.is_available():
        torch.cuda.set_rng_state(rng['cuda'])
    get_rng_tracker().states.update(rng.get('tracker', {}))
    return manifest
