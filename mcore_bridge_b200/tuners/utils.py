"""Sharded-checkpoint description of adapter-wrapped models (parity: reference
``src/mcore_bridge/tuners/utils.py:8-28``, ``src/mcore_bridge/tuners/lora.py:448-474``)."""
from __future__ import annotations

from typing import Dict, List

from torch import nn


def tuners_sharded_state_dict(module: nn.Module, prefix: str = '', sharded_offsets=(),
                              metadata=None) -> Dict[str, List]:
    """The trainable adapter tensors (LoRA factors, ``modules_to_save`` copies) of ``module`` as sharded-checkpoint
    pieces: ``{key: [ShardedTensor, ...]}`` with global shape, this rank's offset and the writer flag, ready for
    ``train.dist_checkpoint.save`` / ``load`` (``trainable_only=True`` does the same for a whole model)."""
    from ..train.dist_checkpoint import sharded_state_dict
    full = sharded_state_dict([module], prefix)
    return {k: v for k, v in full.items() if 'lora_' in k or 'modules_to_save' in k}
