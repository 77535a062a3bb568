"""Hooks ``LoraParallelLinear`` into the real ``peft`` package when it is installed.

``peft.tuners.lora.model.LoraModel._create_new_module`` walks a list of dispatchers; ours wraps the
tensor-parallel linears, grouped expert linears and the router.  Without ``peft`` this module is a no-op and
``tuners.peft_model.get_peft_model`` provides the same behaviour.  Parity: reference
``src/mcore_bridge/tuners/patcher.py:17-62``.
"""
from __future__ import annotations

from ..utils.logger import get_logger

logger = get_logger()
_applied = False


def dispatch_mcb200(target, adapter_name, lora_config, **kwargs):
    from .lora import LoraParallelLinear
    from .peft_model import LORA_TARGET_TYPES
    base = target.base_layer if hasattr(target, 'base_layer') else target
    if isinstance(base, LORA_TARGET_TYPES):
        allowed = ('r', 'lora_alpha', 'lora_dropout', 'fan_in_fan_out', 'init_lora_weights', 'use_rslora', 'use_dora',
                   'lora_bias')
        kw = {k: v for k, v in kwargs.items() if k in allowed}
        return LoraParallelLinear(base_layer=target, adapter_name=adapter_name, **kw)
    return None


def apply_patch() -> bool:
    global _applied
    if _applied:
        return True
    try:
        from peft.tuners.lora import model as lora_model
    except Exception:
        return False
    orig = lora_model.LoraModel._create_new_module

    def _create_new_module(lora_config, adapter_name, target, **kwargs):
        new = dispatch_mcb200(target, adapter_name, lora_config, **kwargs)
        if new is not None:
            return new
        return orig(lora_config, adapter_name, target, **kwargs)

    lora_model.LoraModel._create_new_module = staticmethod(_create_new_module)
    _applied = True
    return True
