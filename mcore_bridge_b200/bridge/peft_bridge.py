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


def _layer_slots(bridge, layer_idx: int, hf_idx: Optional[int] = None) -> List[Tuple[str, str, str, List[str]]]:
    """Every linear of one transformer layer that LoRA may wrap: (path inside the layer, kind, hf prefix relative to
    the layer, hf module names).  ``layer_idx`` selects the layer's structure (MoE or dense, linear or softmax
    attention); ``hf_idx`` is the index the layer has in the checkpoint (MTP layers sit after the decoder)."""
    cfg = bridge.config
    custom = bridge._peft_layer_slots(layer_idx)
    if custom is not None:          # families whose layers are laid out differently give their own table
        return custom
    ap, mp = bridge.hf_attn_prefix + '.', bridge.hf_mlp_prefix + '.'
    lprefix = f'{bridge.hf_layers_prefix}.{layer_idx if hf_idx is None else hf_idx}.'
    slots = []
    if bridge._layer_is_linear_attention(lprefix, 'lightning'):
        slots.append(('self_attention.linear_qkv', 'qkv', ap, ['q_proj', 'k_proj', 'v_proj']))
        slots.append(('self_attention.g_proj', 'column', ap, ['g_proj']))
        slots.append(('self_attention.linear_proj', 'row', ap, ['o_proj']))
    elif cfg.experimental_attention_variant == 'dsv4_hybrid':
        slots.append(('self_attention.linear_q_down_proj', 'replicated', ap, ['wq_a']))
        slots.append(('self_attention.linear_q_up_proj', 'column', ap, ['wq_b']))
        slots.append(('self_attention.linear_kv_proj', 'replicated', ap, ['wkv']))
        slots.append(('self_attention.linear_proj', 'row', ap, ['wo_b']))
    elif cfg.multi_latent_attention:
        if cfg.q_lora_rank is None:
            slots.append(('self_attention.linear_q_proj', 'column', ap, ['q_proj']))
        else:
            slots.append(('self_attention.linear_q_down_proj', 'replicated', ap, ['q_a_proj']))
            slots.append(('self_attention.linear_q_up_proj', 'column', ap, ['q_b_proj']))
        slots.append(('self_attention.linear_kv_down_proj', 'replicated', ap, ['kv_a_proj_with_mqa']))
        slots.append(('self_attention.linear_kv_up_proj', 'column', ap, ['kv_b_proj']))
        slots.append(('self_attention.linear_proj', 'row', ap, ['o_proj']))
        if cfg.experimental_attention_variant == 'dsa':
            ip = ap + 'indexer.'
            slots.append(('self_attention.indexer.linear_wq_b', 'replicated', ip, ['wq_b']))
            slots.append(('self_attention.indexer.linear_wk', 'replicated', ip, ['wk']))
            slots.append(('self_attention.indexer.linear_weights_proj', 'replicated', ip, ['weights_proj']))
    elif bridge._layer_is_linear_attention(lprefix):
        gp = bridge.hf_linear_attn_prefix + '.'
        names = ['in_proj_qkv', 'in_proj_z', 'in_proj_b', 'in_proj_a'] if bridge.split_gdn_projections else \
            ['in_proj_qkvz', 'in_proj_ba']
        slots.append(('self_attention.in_proj', 'gdn_in', gp, names))
        slots.append(('self_attention.out_proj', 'row', gp, ['out_proj']))
    else:
        if bridge.hf_fused_qkv_key is not None:
            slots.append(('self_attention.linear_qkv', 'qkv_fused', ap, [bridge.hf_fused_qkv_key]))
        else:
            slots.append(('self_attention.linear_qkv', 'qkv', ap, ['q_proj', 'k_proj', 'v_proj']))
        slots.append(('self_attention.linear_proj', 'row', ap, [bridge.hf_o_proj_key.rsplit('.', 1)[0]]))
    n_gate, n_up, n_down = bridge.hf_expert_proj_names
    if bridge._layer_is_moe(layer_idx):
        slots.append(('mlp.router', 'replicated', mp, [bridge.hf_gate_key.rsplit('.', 1)[0]]))
        ep = mp + bridge.hf_experts_prefix + '.'
        if cfg.gated_linear_unit:
            slots.append(('mlp.experts.linear_fc1', 'grouped_glu', ep, [n_gate, n_up]))
        else:
            slots.append(('mlp.experts.linear_fc1', 'grouped_col', ep, [n_up]))
        slots.append(('mlp.experts.linear_fc2', 'grouped_row', ep, [n_down]))
        if cfg.moe_shared_expert_intermediate_size:
            sp = mp + bridge.hf_shared_expert_prefix + '.'
            if cfg.gated_linear_unit:
                slots.append(('mlp.shared_experts.linear_fc1', 'glu', sp, ['gate_proj', 'up_proj']))
            else:
                slots.append(('mlp.shared_experts.linear_fc1', 'column', sp, ['up_proj']))
            slots.append(('mlp.shared_experts.linear_fc2', 'row', sp, ['down_proj']))
    else:
        if cfg.gated_linear_unit:
            slots.append(('mlp.linear_fc1', 'glu', mp, ['gate_proj', 'up_proj']))
        else:
            slots.append(('mlp.linear_fc1', 'column', mp, ['up_proj']))
        slots.append(('mlp.linear_fc2', 'row', mp, ['down_proj']))
    return slots


def _mtp_slots(bridge, k: int):
    """(module holding the slot paths, slots, hf layer prefix) for MTP depth ``k``: the projection of the
    concatenated embedding / hidden state plus an ordinary transformer layer, stored after the decoder layers."""
    cfg = bridge.config
    hf_idx = cfg.num_layers + k
    slots = [('eh_proj', 'column', '', ['eh_proj'])]
    slots += [('transformer_layer.' + path, kind, hp, names)
              for path, kind, hp, names in _layer_slots(bridge, cfg.num_layers - 1, hf_idx)]
    return slots, f'{PREFIX}{bridge.hf_layers_prefix}.{hf_idx}.'


def _tp(bridge, is_expert=False):
    name, n, r = bridge._group_info(is_expert)
    return name, n, r


def _gather(bridge, t: Optional[torch.Tensor], tp_dim, is_expert=False):
    t = bridge._all_gather_tp(t, tp_dim, is_expert)
    return bridge._broadcast_pp(t, bridge._device)


def _language_models(bridge, mg_models):
    from ..utils.megatron_utils import unwrap_model
    models = []
    for m in unwrap_model(list(mg_models)):
        while hasattr(m, 'base_model') or (hasattr(m, 'model') and not hasattr(m, 'decoder')):
            m = m.base_model if hasattr(m, 'base_model') else m.model
        models.append(bridge._language_model(m))
    return models


def _iter_layers(bridge, mg_models):
    """Yields ``(module or None, slots, hf key prefix)`` for every decoder layer and then every MTP layer, in the
    same order on every rank (a layer another pipeline stage owns comes as ``None``)."""
    models = _language_models(bridge, mg_models)
    for i in range(bridge.config.num_layers):
        yield bridge._find_layer(models, i), _layer_slots(bridge, i), f'{PREFIX}{bridge.hf_layers_prefix}.{i}.'
    last = next((m for m in models if getattr(m, 'post_process', False)), None)
    mtp = getattr(last, 'mtp', None) if last is not None else None
    for k in range(bridge.config.mtp_num_layers or 0):
        slots, lp = _mtp_slots(bridge, k)
        yield (mtp.layers[k] if mtp is not None else None), slots, lp
    # linears that belong to the model rather than to a layer (family-specific), addressed from the first stage
    extra = bridge._peft_model_slots()
    if extra:
        first = next((m for m in models if getattr(m, 'pre_process', False)), None)
        yield first, extra[0], PREFIX + extra[1]


def _check_all_visited(bridge, mg_models, visited: set, adapter_name: str, what: str) -> None:
    """Raises if the model holds a LoRA-wrapped linear that the slot tables do not describe: its trained factors
    would otherwise be dropped (export) or left at their initial values (load) without a word."""
    Lora = _lora_cls()
    missing = []
    for m in _language_models(bridge, mg_models):
        for name, mod in m.named_modules():
            if isinstance(mod, Lora) and adapter_name in mod.lora_A and id(mod) not in visited:
                missing.append(name)
    if missing:
        raise NotImplementedError(f'adapter {what}: no Hugging Face mapping for the LoRA modules {sorted(missing)[:8]}'
                                  f'{" ..." if len(missing) > 8 else ""}')


def _modules_to_save(bridge, models) -> Iterator[Tuple[str, nn.Module]]:
    return iter(())


def _qkv_rows(cfg):
    d = cfg.kv_channels
    return d * cfg.num_attention_heads // cfg.num_query_groups * (2 if cfg.attention_output_gate else 1), d


def export_adapter(bridge, mg_models, adapter_name: str = 'default') -> Iterator[Tuple[str, torch.Tensor]]:
    Lora = _lora_cls()
    cfg = bridge.config
    out: Dict[str, torch.Tensor] = {}
    visited = set()
    for layer, slots, lp in _iter_layers(bridge, mg_models):
        for path, kind, hp, names in slots:
            mod = deep_getattr(layer, path) if layer is not None else None
            is_lora = isinstance(mod, Lora) and adapter_name in mod.lora_A
            if is_lora:
                visited.add(id(mod))
            if not bridge._agree(is_lora, bridge._device):
                continue
            a = mod.lora_A[adapter_name].weight if is_lora else None
            b = mod.lora_B[adapter_name].weight if is_lora else None
            if kind in ('column', 'replicated', 'qkv', 'qkv_fused', 'glu', 'gdn_in', 'custom_col'):
                A = _gather(bridge, None if a is None else a.detach(), None)
                B = _gather(bridge, None if b is None else b.detach(), None if kind == 'replicated' else
                            ('glu' if kind == 'glu' else 0))
                if A is None:
                    continue
                if kind == 'qkv':
                    parts = qkv_to_hf(B, cfg.num_query_groups, *_qkv_rows(cfg))
                elif kind == 'qkv_fused':
                    parts = [torch.cat(list(qkv_to_hf(B, cfg.num_query_groups, *_qkv_rows(cfg))), dim=0)]
                elif kind == 'glu':
                    parts = B.chunk(2, dim=0)
                elif kind == 'gdn_in':
                    from .gpt_bridge import gdn_in_proj_to_hf
                    by_name = gdn_in_proj_to_hf(B, cfg, bridge.split_gdn_projections)
                    parts = [by_name[n] for n in names]
                elif kind == 'custom_col':
                    parts = bridge._peft_split(lp, path, B, names)
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
    _check_all_visited(bridge, mg_models, visited, adapter_name, 'export')
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
    visited = set()

    def get(key):
        for k in (key, key.replace('.lora_A.weight', f'.lora_A.{adapter_name}.weight').replace(
                '.lora_B.weight', f'.lora_B.{adapter_name}.weight')):
            if k in sd:
                return sd[k].load()
        raise KeyError(f'{key} is missing from the adapter checkpoint')

    for layer, slots, lp in _iter_layers(bridge, mg_models):
        if layer is None:
            continue
        for path, kind, hp, names in slots:
            mod = deep_getattr(layer, path)
            if not (isinstance(mod, Lora) and adapter_name in mod.lora_A):
                continue
            visited.add(id(mod))
            a, b = mod.lora_A[adapter_name].weight, mod.lora_B[adapter_name].weight
            is_expert = mod.is_expert
            _, n, r = _tp(bridge, is_expert)
            if kind in ('column', 'replicated', 'qkv', 'qkv_fused', 'glu', 'gdn_in', 'custom_col'):
                As = [get(f'{lp}{hp}{nm}.lora_A.weight') for nm in names]
                for other in As[1:]:
                    assert torch.equal(As[0], other), f'{path}: the fused projections need identical lora_A matrices'
                Bs = [get(f'{lp}{hp}{nm}.lora_B.weight') for nm in names]
                if kind == 'qkv':
                    B, tp_dim = qkv_to_mcore(*Bs, cfg.num_query_groups), 0
                elif kind == 'qkv_fused':
                    q_rows, d = _qkv_rows(cfg)
                    nq, nkv = q_rows * cfg.num_query_groups, d * cfg.num_query_groups
                    w = Bs[0]
                    B, tp_dim = qkv_to_mcore(w[:nq], w[nq:nq + nkv], w[nq + nkv:], cfg.num_query_groups), 0
                elif kind == 'glu':
                    B, tp_dim = torch.cat(Bs, dim=0), 'glu'
                elif kind == 'gdn_in':
                    from .gpt_bridge import gdn_in_proj_to_mcore
                    B, tp_dim = gdn_in_proj_to_mcore(dict(zip(names, Bs)), cfg, bridge.split_gdn_projections), 0
                elif kind == 'custom_col':
                    B, tp_dim = bridge._peft_join(lp, path, Bs, names), 0
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
    _check_all_visited(bridge, mg_models, visited, adapter_name, 'load')


def hf_target_modules(bridge, mg_models, adapter_name: str = 'default') -> List[str]:
    """Hugging Face module names of every wrapped linear.  Under pipeline parallelism the names are gathered over
    the pipeline group, so every rank of that group has to call this (``GPTBridge.save_weights`` does)."""
    Lora = _lora_cls()
    found = set()
    for layer, slots, _ in _iter_layers(bridge, mg_models):
        if layer is None:
            continue
        for path, kind, hp, names in slots:
            mod = deep_getattr(layer, path)
            if isinstance(mod, Lora) and adapter_name in mod.lora_A:
                found.update(names)
    if dist.is_available() and dist.is_initialized() and ps.get_world_size('pp') > 1:
        gathered = [None] * ps.get_world_size('pp')
        dist.all_gather_object(gathered, sorted(found), group=ps.get_group('pp'))
        for g in gathered:
            found.update(g)
    return sorted(found)


def save_adapter_config(bridge, mg_models, output_dir: str, adapter_name: str = 'default',
                        target_modules: Optional[List[str]] = None) -> None:
    """Writes ``adapter_config.json`` with Hugging Face module names as ``target_modules`` (the reference leaves
    this to the user, ``README.md:281-284``; here it is derived from the wrapped modules).  Called on one rank only:
    under pipeline parallelism pass ``target_modules`` collected beforehand by :func:`hf_target_modules` on every
    rank, because collecting them is a collective."""
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
    if target_modules is None:
        target_modules = hf_target_modules(bridge, mg_models, adapter_name)
    cfg_dict['target_modules'] = target_modules
    cfg_dict['modules_to_save'] = None if not cfg_dict.get('modules_to_save') else cfg_dict['modules_to_save']
    os.makedirs(output_dir, exist_ok=True)
    with open(os.path.join(output_dir, 'adapter_config.json'), 'w') as f:
        json.dump(cfg_dict, f, indent=2, default=lambda o: sorted(o) if isinstance(o, set) else str(o))
