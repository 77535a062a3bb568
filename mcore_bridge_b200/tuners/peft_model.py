"""Minimal PEFT-compatible LoRA injection (``LoraConfig`` / ``get_peft_model``) for environments without ``peft``.

Behaviour follows PEFT where the weight bridge and user scripts depend on it: target matching (a regex for a
string, suffix match for a list, ``'all-linear'``), freezing of the base model, ``modules_to_save`` copies, the
``base_model.model.`` key prefix and ``adapter_config.json`` fields.  When the real ``peft`` package is present,
``tuners/patcher.py`` registers ``LoraParallelLinear`` with its dispatcher instead, so ``peft.get_peft_model``
works on our models (parity: reference ``src/mcore_bridge/tuners/patcher.py:17-56``).
"""
from __future__ import annotations

import copy
import json
import os
import re
from dataclasses import asdict, dataclass
from typing import List, Optional, Union

from torch import nn

from ..layers.linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
from ..layers.moe import GroupedLinear, TopKRouter
from ..utils.utils import patch_deepcopy
from .lora import LoraParallelLinear

LORA_TARGET_TYPES = (ColumnParallelLinear, RowParallelLinear, GroupedLinear, TopKRouter, ReplicatedLinear)


@dataclass
class LoraConfig:
    r: int = 8
    lora_alpha: int = 8
    target_modules: Optional[Union[List[str], str]] = None
    exclude_modules: Optional[Union[List[str], str]] = None
    lora_dropout: float = 0.0
    fan_in_fan_out: bool = False
    bias: str = 'none'
    use_rslora: bool = False
    use_dora: bool = False
    modules_to_save: Optional[List[str]] = None
    init_lora_weights: Union[bool, str] = True
    lora_bias: bool = False
    task_type: Optional[str] = 'CAUSAL_LM'
    peft_type: str = 'LORA'
    base_model_name_or_path: Optional[str] = None
    inference_mode: bool = False

    def to_dict(self) -> dict:
        d = asdict(self)
        if isinstance(d.get('target_modules'), (set, tuple)):
            d['target_modules'] = sorted(d['target_modules'])
        return d


def _matches(name: str, spec) -> bool:
    if spec is None:
        return False
    if isinstance(spec, str):
        return re.fullmatch(spec, name) is not None
    return any(name == t or name.endswith('.' + t) for t in spec)


class ModulesToSaveWrapper(nn.Module):
    """Keeps the frozen original and a trainable copy per adapter (PEFT's ``modules_to_save``)."""

    def __init__(self, module: nn.Module, adapter_name: str):
        super().__init__()
        self.original_module = module
        self.modules_to_save = nn.ModuleDict()
        self._active_adapter = adapter_name
        self.update(adapter_name)

    def update(self, adapter_name: str):
        with patch_deepcopy():
            clone = copy.deepcopy(self.original_module)
        for (n, p), (_, q) in zip(clone.named_parameters(), self.original_module.named_parameters()):
            for attr in ('tensor_model_parallel', 'partition_dim', 'partition_stride', 'sequence_parallel', 'is_expert',
                         'allreduce'):
                if hasattr(q, attr):
                    setattr(p, attr, getattr(q, attr))
            p.requires_grad_(True)
        self.original_module.requires_grad_(False)
        self.modules_to_save[adapter_name] = clone

    @property
    def weight(self):
        return self.modules_to_save[self._active_adapter].weight

    def forward(self, *args, **kwargs):
        return self.modules_to_save[self._active_adapter](*args, **kwargs)


class LoraModel(nn.Module):

    def __init__(self, model: nn.Module, config: LoraConfig, adapter_name: str = 'default'):
        super().__init__()
        self.model = model
        self.peft_config = {adapter_name: config}
        self.active_adapter = adapter_name
        self.targeted_module_names: List[str] = []
        self._inject(config, adapter_name)
        self._mark_trainable(adapter_name)

    def _inject(self, cfg: LoraConfig, adapter_name: str):
        target = cfg.target_modules
        names = [n for n, _ in self.model.named_modules()]
        for name in names:
            parent_name, _, child = name.rpartition('.')
            try:
                parent = self.model.get_submodule(parent_name) if parent_name else self.model
                module = getattr(parent, child)
            except AttributeError:
                continue
            if isinstance(module, LoraParallelLinear) or '.lora_' in name or '.base_layer' in name:
                continue
            if cfg.modules_to_save and _matches(name, cfg.modules_to_save) \
                    and not isinstance(module, ModulesToSaveWrapper):
                setattr(parent, child, ModulesToSaveWrapper(module, adapter_name))
                continue
            if not isinstance(module, LORA_TARGET_TYPES):
                continue
            if cfg.exclude_modules and _matches(name, cfg.exclude_modules):
                continue
            if target == 'all-linear':
                hit = not isinstance(module, TopKRouter) and not name.endswith('output_layer')
            else:
                hit = _matches(name, target)
            if not hit:
                continue
            wrapped = LoraParallelLinear(module, adapter_name, r=cfg.r, lora_alpha=cfg.lora_alpha,
                                         lora_dropout=cfg.lora_dropout, fan_in_fan_out=cfg.fan_in_fan_out,
                                         init_lora_weights=cfg.init_lora_weights, use_rslora=cfg.use_rslora,
                                         use_dora=cfg.use_dora, lora_bias=cfg.lora_bias)
            setattr(parent, child, wrapped)
            self.targeted_module_names.append(name)
        if not self.targeted_module_names and not cfg.modules_to_save:
            raise ValueError(f'Target modules {target} not found in the base model.')

    def _mark_trainable(self, adapter_name: str):
        for n, p in self.model.named_parameters():
            trainable = ('lora_' in n) or ('modules_to_save' in n)
            p.requires_grad_(trainable)

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            if name == 'model':
                raise
            return getattr(self.model, name)

    def merge_adapter(self):
        for m in self.model.modules():
            if isinstance(m, LoraParallelLinear):
                m.merge()

    def unmerge_adapter(self):
        for m in self.model.modules():
            if isinstance(m, LoraParallelLinear):
                m.unmerge()


class PeftModel(nn.Module):
    """``peft.PeftModel`` look-alike: parameters live under ``base_model.model.``."""

    def __init__(self, model: nn.Module, config: LoraConfig, adapter_name: str = 'default'):
        super().__init__()
        self.base_model = LoraModel(model, config, adapter_name)
        self.peft_config = self.base_model.peft_config
        self.active_adapter = adapter_name

    def forward(self, *args, **kwargs):
        return self.base_model(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            if name == 'base_model':
                raise
            return getattr(self.base_model, name)

    def get_base_model(self):
        return self.base_model.model

    def print_trainable_parameters(self):
        t = sum(p.numel() for p in self.parameters() if p.requires_grad)
        a = sum(p.numel() for p in self.parameters())
        print(f'trainable params: {t:,} || all params: {a:,} || trainable%: {100 * t / max(a, 1):.4f}')

    def save_config(self, output_dir: str, adapter_name: Optional[str] = None, target_modules=None):
        cfg = self.peft_config[adapter_name or self.active_adapter].to_dict()
        if target_modules is not None:
            cfg['target_modules'] = target_modules
        os.makedirs(output_dir, exist_ok=True)
        with open(os.path.join(output_dir, 'adapter_config.json'), 'w') as f:
            json.dump(cfg, f, indent=2, default=str)


def get_peft_model(model: nn.Module, peft_config: LoraConfig, adapter_name: str = 'default') -> PeftModel:
    return PeftModel(model, peft_config, adapter_name)
