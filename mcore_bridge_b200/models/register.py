"""Model registry and factory.

``register_model(ModelMeta)`` maps Hugging Face ``model_type`` strings to a model class, a bridge class and
(for multimodal families) a vision-tower class; ``get_mcore_model(config)`` builds the model chunk(s) this
pipeline rank owns — one per virtual stage under interleaved pipelining, with ``pre_process`` /
``post_process`` taken from the stage position.  Parity: reference ``src/mcore_bridge/model/register.py:33-235``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Type

import torch
from torch import nn

from ..parallel import state as ps
from ..utils.logger import get_logger

logger = get_logger()
MODEL_MAPPING: Dict[str, 'ModelMeta'] = {}
_hf_to_mcore: Optional[Dict[str, str]] = None


@dataclass
class ModelMeta:
    model_type: str
    model_types: List[str]
    bridge_cls: Optional[Type] = None
    visual_cls: Optional[Type[nn.Module]] = None
    is_multimodal: bool = False
    loader: Optional[Type['ModelLoader']] = None

    def __post_init__(self):
        if self.bridge_cls is None:
            from ..bridge.gpt_bridge import GPTBridge
            self.bridge_cls = GPTBridge
        if self.visual_cls is not None:
            self.is_multimodal = True
        if self.loader is None:
            self.loader = ModelLoader


def register_model(model_meta: ModelMeta, *, exist_ok: bool = False):
    global _hf_to_mcore
    if not exist_ok and model_meta.model_type in MODEL_MAPPING:
        raise ValueError(f'The `{model_meta.model_type}` has already been registered in the MODEL_MAPPING.')
    MODEL_MAPPING[model_meta.model_type] = model_meta
    _hf_to_mcore = None


def _ensure_families_loaded():
    from . import gpts, mm_gpts  # noqa: F401  (registration happens at import)


def get_mcore_model_type(hf_model_type: Optional[str]) -> Optional[str]:
    global _hf_to_mcore
    _ensure_families_loaded()
    if _hf_to_mcore is None:
        _hf_to_mcore = {}
        for k, meta in MODEL_MAPPING.items():
            for t in meta.model_types:
                _hf_to_mcore[t] = k
    res = _hf_to_mcore.get(hf_model_type)
    if res is None:
        raise ValueError(f'unsupported hf_model_type {hf_model_type!r}; registered: {sorted(_hf_to_mcore)}')
    return res


def get_model_meta(mcore_model_type: str) -> ModelMeta:
    _ensure_families_loaded()
    return MODEL_MAPPING[mcore_model_type]


class ModelLoader:
    """Builds one model chunk.  Families override ``model_cls`` or ``build_model`` to swap modules."""
    model_cls = None

    def __init__(self, config):
        self.config = config

    def get_model_cls(self):
        if self.model_cls is not None:
            return self.model_cls
        if self.config.is_multimodal and not self.config.language_model_only:
            from .mm_gpt_model import MultimodalGPTModel
            return MultimodalGPTModel
        from .gpt_model import GPTModel
        return GPTModel

    def build_model(self, pre_process: bool = True, post_process: bool = True, vp_stage: Optional[int] = None):
        cfg = self.config
        device = torch.device('cuda', torch.cuda.current_device()) if torch.cuda.is_available() else torch.device('cpu')
        with torch.device(device):
            model = self.get_model_cls()(cfg, pre_process=pre_process, post_process=post_process, vp_stage=vp_stage)
        return model


def get_mcore_model(config) -> List[nn.Module]:
    """One model chunk per virtual pipeline stage owned by this rank (a list of length 1 without VPP)."""
    loader = config.model_meta.loader(config)
    vpp = config.virtual_pipeline_model_parallel_size
    models = []
    if ps.get_pipeline_model_parallel_world_size() > 1 and vpp is not None and vpp > 1:
        for i in range(vpp):
            pre = ps.is_pipeline_first_stage(ignore_virtual=False, vp_stage=i)
            post = ps.is_pipeline_last_stage(ignore_virtual=False, vp_stage=i)
            models.append(loader.build_model(pre, post, vp_stage=i))
    else:
        models.append(loader.build_model(ps.is_pipeline_first_stage(), ps.is_pipeline_last_stage()))
    return models
