"""Lazy safetensors reader and streaming, size-bounded safetensors writer.

File naming matches Hugging Face conventions so Transformers can load the result:
``model.safetensors`` for one shard, else ``model-XXXXX-of-YYYYY.safetensors`` plus
``model.safetensors.index.json`` with ``metadata.total_size``; PEFT adapters go to a single
``adapter_model.safetensors``.  Parity: reference ``src/mcore_bridge/utils/safetensors.py:24-168``.

The writer hands finished shards to a background thread, so serialisation overlaps with the
gather/convert work of the next tensors.
"""
from __future__ import annotations

import json
import os
import queue
import re
import threading
from typing import Dict, Literal, Optional

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from .env import is_last_rank, is_master


class LazyTensor:
    """A tensor that is read from disk only when :meth:`load` is called."""

    def __init__(self, tensor: Optional[torch.Tensor] = None, loader=None):
        self.tensor = tensor
        self.loader = loader

    def load(self) -> torch.Tensor:
        if self.tensor is None:
            return self.loader()
        return self.tensor


class SafetensorLazyLoader:

    def __init__(self, hf_model_dir: str, peft_format: bool = False):
        self.hf_model_dir = hf_model_dir
        self.peft_format = peft_format
        self._handles = {}
        self._weight_map: Dict[str, str] = {}
        self._load_index()

    def _open_file(self, filename: str):
        h = self._handles.get(filename)
        if h is None:
            h = safe_open(os.path.join(self.hf_model_dir, filename), framework='pt', device='cpu')
            self._handles[filename] = h
        return h

    def _load_index(self):
        d = self.hf_model_dir
        if self.peft_format:
            files = ['adapter_model.safetensors']
        else:
            index_path = os.path.join(d, 'model.safetensors.index.json')
            if os.path.exists(index_path):
                with open(index_path, 'r', encoding='utf-8') as f:
                    self._weight_map = dict(json.load(f)['weight_map'])
                return
            if os.path.exists(os.path.join(d, 'model.safetensors')):
                files = ['model.safetensors']
            else:
                files = sorted(f for f in os.listdir(d) if f.endswith('.safetensors'))
                if not files:
                    raise FileNotFoundError(f'no safetensors files in {d}')
        for fn in files:
            for key in self._open_file(fn).keys():
                self._weight_map[key] = fn

    def keys(self):
        return self._weight_map.keys()

    def get_state_dict(self) -> Dict[str, LazyTensor]:
        return {k: LazyTensor(loader=(lambda k=k: self._load_tensor(k))) for k in self._weight_map}

    def _load_tensor(self, key: str) -> torch.Tensor:
        return self._open_file(self._weight_map[key]).get_tensor(key)

    def get_slice(self, key: str):
        return self._open_file(self._weight_map[key]).get_slice(key)

    def close(self):
        self._handles.clear()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.close()


def _parse_size(s) -> int:
    if isinstance(s, (int, float)):
        return int(s)
    m = re.fullmatch(r'\s*([\d.]+)\s*(GB|MB|KB|B)?\s*', s, flags=re.I)
    if not m:
        raise ValueError(f'Invalid max_shard_size: {s}')
    mult = {'GB': 1000**3, 'MB': 1000**2, 'KB': 1000, 'B': 1, None: 1}[m.group(2).upper() if m.group(2) else None]
    return int(float(m.group(1)) * mult)


class StreamingSafetensorSaver:

    def __init__(self, save_dir, max_shard_size='5GB', save_rank: Literal['master', 'last'] = 'master',
                 peft_format: bool = False, background: bool = True) -> None:
        self.save_dir = save_dir
        self.max_shard_size = _parse_size(max_shard_size)
        self.current_shard: Dict[str, torch.Tensor] = {}
        self.current_shard_size = 0
        self.total_size = 0
        self.shard_index = 1
        self.weight_map: Dict[str, str] = {}
        self.is_save_rank = is_master() if save_rank == 'master' else is_last_rank()
        self.peft_format = peft_format
        self._q: Optional[queue.Queue] = None
        self._thread = None
        self._error = None
        if self.is_save_rank:
            os.makedirs(save_dir, exist_ok=True)
            if background:
                self._q = queue.Queue(maxsize=2)
                self._thread = threading.Thread(target=self._writer, daemon=True)
                self._thread.start()

    def _writer(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            shard, path = item
            try:
                save_file(shard, path, metadata={'format': 'pt'})
            except Exception as e:  # surfaced in finalize
                self._error = e

    def add_tensor(self, name: str, tensor: torch.Tensor):
        if not self.is_save_rank:
            return
        size = tensor.numel() * tensor.element_size()
        if self.current_shard and not self.peft_format and self.current_shard_size + size > self.max_shard_size:
            self._save_current_shard()
        self.current_shard[name] = tensor.detach().cpu().contiguous()
        self.current_shard_size += size

    def _save_current_shard(self, shard_filename: Optional[str] = None):
        if not self.current_shard:
            return
        if shard_filename is None:
            shard_filename = ('adapter_model.safetensors' if self.peft_format else
                              f'model-{self.shard_index:05d}-of-?????.safetensors')
        path = os.path.join(self.save_dir, shard_filename)
        if self._q is not None:
            self._q.put((self.current_shard, str(path)))
        else:
            save_file(self.current_shard, str(path), metadata={'format': 'pt'})
        for key in self.current_shard:
            self.weight_map[key] = shard_filename
        self.total_size += self.current_shard_size
        self.current_shard = {}
        self.current_shard_size = 0
        self.shard_index += 1

    def finalize(self):
        if not self.is_save_rank:
            return
        if self.current_shard:
            self._save_current_shard()
        if self._q is not None:
            self._q.put(None)
            self._thread.join()
            if self._error is not None:
                raise self._error
        if self.peft_format:
            return
        total = self.shard_index - 1
        for i in range(1, total + 1):
            old = os.path.join(self.save_dir, f'model-{i:05d}-of-?????.safetensors')
            new_name = 'model.safetensors' if total == 1 else f'model-{i:05d}-of-{total:05d}.safetensors'
            if os.path.exists(old):
                os.replace(old, os.path.join(self.save_dir, new_name))
        if total > 1:
            wm = {k: v.replace('?????', f'{total:05d}') for k, v in self.weight_map.items()}
            with open(os.path.join(self.save_dir, 'model.safetensors.index.json'), 'w') as f:
                json.dump({'metadata': {'total_size': self.total_size}, 'weight_map': wm}, f, indent=2)
