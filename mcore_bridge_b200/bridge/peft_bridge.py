"""PEFT-format (``adapter_model.safetensors`` + ``adapter_config.json``) import / export of LoRA adapters.

Key naming is the one Transformers + PEFT expect: ``base_model.model.<hf module path>.lora_A.weight`` /
``.lora_B.weight`` (the adapter name is not part of the saved key) and, for ``modules_to_save``, the plain
HF weight key under ``base_model.model.``.  Re-layouts mirror the full-weight bridge (parity: reference
``src/mcore_bridge/bridge/gpt_bridge.py:254-329,473-495,549-624,977-1031``):

* fused QKV: ``lora_A`` is shared by q/k/v (load asserts the three HF copies are equal), ``lora_B`` is
  interleaved per query group exactly like the weight;
* fused gate/up: shared ``lora_A``, ``lora_B`` stacked ``[gate; up]``;
* row-parallel layers: ``lora_A`` is sharded on its input dim, ``lora_B`` replicated;
* experts: one key set per expert from the stacked factors.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterator, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from ..parallel import state as ps
from ..utils.safetensors import LazyTensor
from ..utils.utils import deep_getattr
from .gpt_bridge import qkv_to_hf, qkv_to_mcore, shard

PREFIX = 'base_model.model.'


def _lora_cls():
    from ..tuners.lora import LoraParallelLinear
    return LoraParallelLinear


def _layer_slots(bridge, layer_idx: int) -> List[Tuple[str, str, str, List[str]]]:
    """(path inside the layer, kind, hf prefix relative to the layer, hf module names)."""
    cfg = bridge.config
    ap, mp = bridge.hf_attn_prefix + '.', bridge.hf_mlp_prefix + '.'
    slots = []
    if cfg.multi_latent_attention:
        if cfg.q_lora_rank is None:
            slots.append(('self_attention.linear_q_proj', 'column', ap, ['q_proj']))
        else:
            slots.append(('self_attention.linear_q_down_proj', 'replicated', ap, ['q_a_proj']))
            slots.append(('self_attention.linear_q_up_proj', 'column', ap, ['q_b_proj']))
        slots.append(('self_attention.linear_kv_down_proj', 'replicated', ap, ['kv_a_proj_with_mqa']))
        slots.append(('self_attention.linear_kv_up_proj', 'column', ap, ['kv_b_proj']))
    else:
        slots.append(('self_attention.linear_qkv', 'qkv', ap, ['q_proj', 'k_proj', 'v_proj']))
    slots.append(('self_attention.linear_proj', 'row', ap, ['o_proj']))
    if bridge._layer_is_moe(layer_idx):
        slots.append(('mlp.router', 'replicated', mp, ['gate']))
        slots.append(('mlp.experts.linear_fc1', 'grouped_glu', mp + bridge.hf_experts_prefix + '.', ['gate_proj', 'up_proj']))
        slots.append(('mlp.experts.linear_fc2', 'grouped_row', mp + bridge.hf_experts_prefix + '.', ['down_proj']))
        if cfg.moe_shared_expert_intermediate_size:
            sp = mp + bridge.hf_shared_expert_prefix + '.'
            slots.append(('mlp.shared_experts.linear_fc1', 'glu', sp, ['gate_proj', 'up_proj']))
            slots.append(('mlp.shared_experts.linear_fc2', 'row', sp, ['down_proj']))
    else:
        if cfg.gated_linear_unit:
            slots.append(('mlp.linear_fc1', 'glu', mp, ['gate_proj', 'up_proj']))
        else:
            slots.append(('mlp.linear_fc1', 'column', mp, ['up_proj']))
        slots.append(('mlp.linear_fc2', 'row', mp, ['down_proj']))
    return slots


def _tp(bridge, is_expert=False):
    name, n, r = bridge._group_info(is_expert)
    return name, n, r


def _gather(bridge, t: Optional[torch.Tensor], tp_dim, is_expert=False):
    t = bridge._all_gather_tp(t, tp_dim, is_expert)
    return bridge._broadcast_pp(t, bridge._device)


def _iter_layers(bridge, mg_models):
    from ..utils.megatron_utils import unwrap_model
    models = []
    for m in unwrap_model(list(mg_models)):
        while hasattr(m, 'base_model') or (hasattr(m, 'model') and not hasattr(m, 'decoder')):
            m = m.base_model if hasattr(m, 'base_model') else m.model
        models.append(bridge._language_model(m))
    for i in range(bridge.config.num_layers):
        yield i, bridge._find_layer(models, i)
    return


def _modules_to_save(bridge, models) -> Iterator[Tuple[str, nn.Module]]:
    return iter(())


def export_adapter(bridge, mg_models, adapter_name: str = 'default') -> Iterator[Tuple[str, torch.Tensor]]:
    Lora = _lora_cls()
    cfg = bridge.config
    out: Dict[str, torch.Tensor] = {}
    for i, layer in _iter_layers(bridge, mg_models):
        lp = f'{PREFIX}{bridge.hf_layers_prefix}.{i}.'
        for path, kind, hp, names in _layer_slots(bridge, i):
            mod = deep_getattr(layer, path) if layer is not None else None
            is_lora = isinstance(mod, Lora) and adapter_name in mod.lora_A
            if not bridge._agree(is_lora, bridge._device):
                continue
            a = mod.lora_A[adapter_name].weight if is_lora else None
            b = mod.lora_B[adapter_name].weight if is_lora else None
            if kind in ('column', 'replicated', 'qkv', 'glu'):
                A = _gather(bridge, None if a is None else a.detach(), None)
                B = _gather(bridge, None if b is None else b.detach(), None if kind == 'replicated' else
                            ('glu' if kind == 'glu' else 0))
                if A is None:
                    continue
                if kind == 'qkv':
                    d = cfg.kv_channels
                    q_rows = d * cfg.num_attention_heads // cfg.num_query_groups * (2 if cfg.attention_output_gate else 1)
                    parts = qkv_to_hf(B, cfg.num_query_groups, q_rows, d)
                elif kind == 'glu':
                    parts = B.chunk(2, dim=0)
                else:
                    parts = [B]
                for n, bp in zip(names, parts):
                    bridge._emit(out, f'{lp}{hp}{n}.lora_A.weight', A)
                    bridge._emit(out, f'{lp}{hp}{n}.lora_B.weight', bp)
            elif kind == 'row':
                A = _gather(bridge, None if a is None else a.detach(), 1)
                B = _gather(bridge, None if b is None else b.detach(), None)
                if A is None:
                    continue
                bridge._emit(out, f'{lp}{hp}{names[0]}.lora_A.weight', A)
                bridge._emit(out, f'{lp}{hp}{names[0]}.lora_B.weight', B)
            else:  # grouped experts: stacked [E_local, ...] -> all experts
                A = bridge._broadcast_pp(bridge._all_gather_ep(None if a is None else a.detach()), bridge._device)
                B = bridge._broadcast_pp(bridge._all_gather_ep(None if b is None else b.detach()), bridge._device)
                if A is None:
                    continue
                for e in range(A.shape[0]):
                    parts = B[e].chunk(2, dim=0) if kind == 'grouped_glu' else [B[e]]
                    for n, bp in zip(names, parts):
                        bridge._emit(out, f'{lp}{hp}{e}.{n}.lora_A.weight', A[e])
                        bridge._emit(out, f'{lp}{hp}{e}.{n}.lora_B.weight', bp)
        for k, v in list(out.items()):
            yield k, v
        out.clear()
    # modules_to_save: export the trainable copies under their plain HF names
    from ..tuners.peft_model import ModulesToSaveWrapper
    from ..utils.megatron_utils import unwrap_model
    for m in unwrap_model(list(mg_models)):
        wrappers = {n: w for n, w in m.named_modules() if isinstance(w, ModulesToSaveWrapper)}
        if not wrappers:
            continue
        inner = m
        while hasattr(inner, 'base_model') or (hasattr(inner, 'model') and not hasattr(inner, 'decoder')):
            inner = inner.base_model if hasattr(inner, 'base_model') else inner.model
        for k, v in bridge._convert_modules_to_save(inner, adapter_name):
            yield PREFIX + k, v


def load_adapter(bridge, mg_models, sd: Dict[str, LazyTensor], adapter_name: str = 'default') -> None:
    Lora = _lora_cls()
    cfg = bridge.config

    def get(key):
        for k in (key, key.replace('.lora_A.weight', f'.lora_A.{adapter_name}.weight').replace(
                '.lora_B.weight', f'.lora_B.{adapter_name}.weight')):
            if k in sd:
                return sd[k].load()
        raise KeyError(f'{key} is missing from the adapter checkpoint')

    for i, layer in _iter_layers(bridge, mg_models):
        if layer is None:
            continue
        lp = f'{PREFIX}{bridge.hf_layers_prefix}.{i}.'
        for path, kind, hp, names in _layer_slots(bridge, i):
            mod = deep_getattr(layer, path)
            if not (isinstance(mod, Lora) and adapter_name in mod.lora_A):
                continue
            a, b = mod.lora_A[adapter_name].weight, mod.lora_B[adapter_name].weight
            is_expert = mod.is_expert
            _, n, r = _tp(bridge, is_expert)
            if kind in ('column', 'replicated', 'qkv', 'glu'):
                As = [get(f'{lp}{hp}{nm}.lora_A.weight') for nm in names]
                for other in As[1:]:
                    assert torch.equal(As[0], other), f'{path}: the fused projections need identical lora_A matrices'
                Bs = [get(f'{lp}{hp}{nm}.lora_B.weight') for nm in names]
                if kind == 'qkv':
                    B = qkv_to_mcore(*Bs, cfg.num_query_groups)
                    tp_dim = 0
                elif kind == 'glu':
                    B, tp_dim = torch.cat(Bs, dim=0), 'glu'
                else:
                    B, tp_dim = Bs[0], (None if kind == 'replicated' else 0)
                with torch.no_grad():
                    a.copy_(As[0].to(a.dtype))
                    b.copy_(shard(B, tp_dim, r, n).to(b.dtype))
            elif kind == 'row':
                A = get(f'{lp}{hp}{names[0]}.lora_A.weight')
                B = get(f'{lp}{hp}{names[0]}.lora_B.weight')
                with torch.no_grad():
                    a.copy_(shard(A, 1, r, n).to(a.dtype))
                    b.copy_(B.to(b.dtype))
            else:
                ep = ps.get_world_size('ep')
                ep_rank = ps.get_rank_in('ep') if ep > 1 else 0
                El = a.shape[0]
                for le in range(El):
                    e = ep_rank * El + le
                    As = [get(f'{lp}{hp}{e}.{nm}.lora_A.weight') for nm in names]
                    for other in As[1:]:
                        assert torch.equal(As[0], other), f'{path}: gate/up need identical lora_A matrices'
                    Bs = [get(f'{lp}{hp}{e}.{nm}.lora_B.weight') for nm in names]
                    with torch.no_grad():
                        a[le].copy_(As[0].to(a.dtype))
                        b[le].copy_(torch.cat(Bs, dim=0).to(b.dtype))


def hf_target_modules(bridge, mg_models, adapter_name: str = 'default') -> List[str]:
    Lora = _lora_cls()
    found = set()
    for i, layer in _iter_layers(bridge, mg_models):
        if layer is None:
            continue
        for path, kind, hp, names in _layer_slots(bridge, i):
            mod = deep_getattr(layer, path)
            if isinstance(mod, Lora) and adapter_name in mod.lora_A:
                found.update(names)
    if dist.is_available() and dist.is_initialized() and ps.get_world_size('pp') > 1:
        gathered = [None] * ps.get_world_size('pp')
        dist.all_gather_object(gathered, sorted(found), group=ps.get_group('pp'))
        for g in gathered:
            found.update(g)
    return sorted(found)


def save_adapter_config(bridge, mg_models, output_dir: str, adapter_name: str = 'default') -> None:
    """Writes ``adapter_config.json`` with Hugging Face module names as ``target_modules`` (the reference leaves
    this to the user, ``README.md:281-284``; here it is derived from the wrapped modules)."""
    from ..utils.megatron_utils import unwrap_model
    cfg_dict = None
    for m in unwrap_model(list(mg_models)):
        pc = getattr(m, 'peft_config', None)
        if pc and adapter_name in pc:
            c = pc[adapter_name]
            cfg_dict = c.to_dict() if hasattr(c, 'to_dict') else dict(c)
            break
    if cfg_dict is None:
        return
    cfg_dict['target_modules'] = hf_target_modules(bridge, mg_models, adapter_name)
    cfg_dict['modules_to_save'] = None if not cfg_dict.get('modules_to_save') else cfg_dict['modules_to_save']
    os.makedirs(output_dir, exist_ok=True)
    with open(os.path.join(output_dir, 'adapter_config.json'), 'w') as f:
        json.dump(cfg_dict, f, indent=2, default=lambda o: sorted(o) if isinstance(o, set) else str(o))
