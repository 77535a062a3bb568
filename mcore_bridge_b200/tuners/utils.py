"""State-dict helpers for adapter-wrapped models (parity: reference ``src/mcore_bridge/tuners/utils.py:8-28``)."""
from __future__ import annotations

from typing import Dict

from torch import nn


def tuners_sharded_state_dict(module: nn.Module, prefix: str = '', sharded_offsets=(), metadata=None) -> Dict[str, dict]:
    """Describes every trainable adapter tensor with its sharding so a sharded checkpoint writer can place it:
    ``{key: {'tensor', 'tp_parallel', 'partition_dim', 'is_expert'}}``."""
    out = {}
    for name, p in module.named_parameters():
        if 'lora_' not in name and 'modules_to_save' not in name:
            continue
        out[prefix + name] = {
            'tensor': p,
            'tp_parallel': bool(getattr(p, 'tensor_model_parallel', False)),
            'partition_dim': int(getattr(p, 'partition_dim', -1)),
            'is_expert': bool(getattr(p, 'is_expert', False)),
        }
    return out
