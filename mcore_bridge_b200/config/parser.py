"""``hf_to_mcore_config``: Hugging Face ``PretrainedConfig`` -> keyword arguments of ``ModelConfig``.

The output keys and per-family rules match the reference parser
(``src/mcore_bridge/config/parser.py:9-276``).  Structure here: one alias table, a generic reader that
recurses into nested text configs, then a list of small family rules applied in order.
"""
from __future__ import annotations

from functools import partial
from typing import Any, Dict, Tuple

import torch.nn.functional as F

from ..utils.utils import get_env_args

# ModelConfig key -> HF attribute names, first hit wins
ALIASES: Dict[str, Tuple[str, ...]] = {
    'num_layers': ('num_hidden_layers',),
    'hidden_size': ('hidden_size',),
    'mlp_ffn_hidden_size': ('intermediate_size_mlp',),
    'ffn_hidden_size': ('intermediate_size',),
    'num_attention_heads': ('num_attention_heads',),
    'num_query_groups': ('num_key_value_heads',),
    'max_position_embeddings': ('max_position_embeddings',),
    'layernorm_epsilon': ('rms_norm_eps',),
    'rotary_base': ('rope_theta',),
    'padded_vocab_size': ('vocab_size',),
    'attention_dropout': ('attention_dropout',),
    'untie_embeddings_and_output_weights': ('tie_word_embeddings',),
    'swiglu': ('hidden_act',),
    'add_qkv_bias': ('attention_bias', 'qkv_bias', 'use_bias'),
    'add_bias_linear': ('mlp_bias',),
    'kv_channels': ('head_dim',),
    'hf_model_type': ('model_type',),
    'moe_ffn_hidden_size': ('moe_intermediate_size',),
    'moe_shared_expert_intermediate_size': ('shared_expert_intermediate_size',),
    'moe_router_topk': ('num_experts_per_tok', 'moe_topk', 'moe_k', 'top_k_experts'),
    'moe_router_num_groups': ('n_group',),
    'moe_router_group_topk': ('topk_group',),
    'num_moe_experts': ('num_experts', 'n_routed_experts', 'moe_num_experts', 'num_local_experts'),
    'moe_router_pre_softmax': ('norm_topk_prob',),
    'moe_router_enable_expert_bias': ('moe_router_enable_expert_bias',),
    'rotary_interleaved': ('rope_interleave',),
    'q_lora_rank': ('q_lora_rank',),
    'kv_lora_rank': ('kv_lora_rank',),
    'moe_router_score_function': ('scoring_func', 'moe_router_use_sigmoid', 'score_function'),
    'moe_router_bias_update_rate': ('aux_loss_alpha',),
    'qk_head_dim': ('qk_nope_head_dim',),
    'qk_pos_emb_head_dim': ('qk_rope_head_dim',),
    'v_head_dim': ('v_head_dim',),
    'moe_router_topk_scaling_factor': ('routed_scaling_factor', 'router_scaling_factor'),
    'qk_layernorm': ('use_qk_norm', 'qk_norm'),
    'linear_attention_freq': ('full_attention_interval',),
    'linear_num_key_heads': ('linear_num_key_heads',),
    'linear_num_value_heads': ('linear_num_value_heads',),
    'linear_key_head_dim': ('linear_key_head_dim',),
    'linear_value_head_dim': ('linear_value_head_dim',),
    'linear_conv_kernel_dim': ('linear_conv_kernel_dim',),
    'dsa_indexer_n_heads': ('index_n_heads',),
    'dsa_indexer_head_dim': ('index_head_dim',),
    'dsa_indexer_topk': ('index_topk',),
    'dsa_indexer_rotary_interleaved': ('indexer_rope_interleave',),
    'csa_compress_ratios': ('compress_rates',),
    'csa_compress_rotary_base': ('compress_rope_theta',),
    'o_groups': ('o_groups',),
    'o_lora_rank': ('o_lora_rank',),
    'num_residual_streams': ('hc_mult',),
    'mhc_sinkhorn_iterations': ('hc_sinkhorn_iters',),
    'moe_n_hash_layers': ('mlp_layer_types',),
    'activation_func_clamp_value': ('swiglu_limit',),
    'original_max_position_embeddings': ('original_max_position_embeddings',),
    'partial_rotary_factor': ('partial_rotary_factor',),
    'first_k_dense_replace': ('first_k_dense_replace', 'moe_layer_start_index'),
    'n_shared_experts': ('n_shared_experts', 'num_shared_expert', 'moe_num_shared_experts', 'num_shared_experts'),
    'window_size': ('sliding_window',),
    'layer_types': ('layer_types',),
    'interleave_moe_layer_step': ('interleave_moe_layer_step',),
}
# alias kept for users of the reference name
config_mapping = {k: list(v) for k, v in ALIASES.items()}

_NESTED = ('text_config', 'llm_config', 'thinker_config')
_NEGATED = {'untie_embeddings_and_output_weights', 'moe_router_pre_softmax'}


def _read(config, nested: bool = False) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for key, names in ALIASES.items():
        for name in names:
            val = getattr(config, name, None)
            if val is None:
                continue
            if key == 'rotary_base':
                out[key] = int(val)
            elif key in _NEGATED:
                out[key] = not val
            elif key == 'swiglu':
                if val == 'silu':
                    out[key] = True
            elif name == 'moe_router_use_sigmoid':
                if not val:
                    continue
                out[key] = 'sigmoid'
            else:
                if key in ('q_lora_rank', 'kv_lora_rank'):
                    out['multi_latent_attention'] = True
                out['llm_model_type' if (key == 'hf_model_type' and nested) else key] = val
            break
    untie = out.get('untie_embeddings_and_output_weights')
    for sub in _NESTED:
        if hasattr(config, sub) and getattr(config, sub) is not None:
            out.update(_read(getattr(config, sub), nested=True))
    if untie is not None:  # the outer config decides about tying
        out['untie_embeddings_and_output_weights'] = untie
    rs = getattr(config, 'rope_scaling', None)
    if rs is None:
        rp = getattr(config, 'rope_parameters', None)  # transformers >= 5 name
        if isinstance(rp, dict) and rp.get('rope_type', 'default') != 'default':
            rs = rp
        elif isinstance(rp, dict):
            if 'rotary_base' not in out and rp.get('rope_theta') is not None:
                out['rotary_base'] = int(rp['rope_theta'])
            if rp.get('partial_rotary_factor') is not None and 'partial_rotary_factor' not in out:
                out['partial_rotary_factor'] = rp['partial_rotary_factor']
            if rp.get('mrope_section') is not None:
                rs = rp
    if isinstance(rs, int):
        out['rope_scaling'] = {'factor': rs, 'type': 'linear'}
    elif isinstance(rs, dict):
        out['rope_scaling'] = dict(rs)
    return out


def _tie_from_dict(d: dict):
    tie = d.get('tie_word_embeddings')
    for sub in _NESTED:
        if d.get(sub) is not None:
            v = _tie_from_dict(d[sub])
            if v is not None:
                tie = v
    return tie


def _window_pattern(layer_types) -> str:
    return '[' + ','.join('1' if lt == 'sliding_attention' else '0' for lt in layer_types) + ']'


_DEEPSEEK_LIKE = {'deepseek', 'deepseek_v2', 'deepseek_v3', 'kimi_k2', 'deepseek_v32', 'dots1', 'deepseek_v4'}
_QK_NORM_LLM = {'qwen3', 'qwen3_moe', 'qwen3_next'}
_QK_NORM_HF = {'qwen3_omni_moe', 'qwen3_omni', 'qwen3_vl', 'qwen3_vl_moe', 'qwen3_5', 'qwen3_5_moe',
               'llavaonevision1_5'}


def hf_to_mcore_config(hf_config) -> Dict[str, Any]:
    res = _read(hf_config)
    name_or_path = getattr(hf_config, 'name_or_path', None)
    if name_or_path:
        try:
            from transformers import PretrainedConfig
            tie = _tie_from_dict(PretrainedConfig.get_config_dict(name_or_path)[0])
            if tie is not None:
                res['untie_embeddings_and_output_weights'] = not tie
        except Exception:  # a name without a readable config.json: keep what the object says
            pass
    res['hf_config'] = hf_config
    hf_type = res.get('hf_model_type')
    llm = res.get('llm_model_type') or hf_type
    res['llm_model_type'] = llm

    first_k_dense = res.pop('first_k_dense_replace', None)
    n_shared = res.pop('n_shared_experts', None)
    layer_types = res.pop('layer_types', None)
    mlp_ffn = res.pop('mlp_ffn_hidden_size', None)
    moe_step = res.pop('interleave_moe_layer_step', None)
    window = res.pop('window_size', None)
    hash_layers = res.pop('moe_n_hash_layers', None)
    rope_scaling = res.get('rope_scaling') or {}

    if llm in _QK_NORM_LLM or hf_type in _QK_NORM_HF:
        res['qk_layernorm'] = True
    if llm in {'qwen2_moe', 'qwen3_moe', 'qwen3_next'} or hf_type in {'qwen3_omni_moe', 'qwen3_vl_moe', 'qwen3_5_moe'}:
        res.pop('ffn_hidden_size', None)
        if llm in {'qwen2_moe', 'qwen3_next'} or hf_type == 'qwen3_5_moe':
            res['moe_shared_expert_gate'] = True

    if llm in _DEEPSEEK_LIKE or hf_type == 'kimi_vl':
        if llm != 'deepseek':
            res['qk_layernorm'] = True
        res['moe_router_load_balancing_type'] = 'seq_aux_loss'
        if llm == 'dots1':
            res['moe_router_score_function'] = 'sigmoid'
        if llm in ('deepseek_v3', 'kimi_k2', 'deepseek_v32'):
            # these architectures always route with sigmoid scores; a config that leaves `scoring_func` out (the
            # Transformers config class has no such field) must not fall back to softmax
            res.setdefault('moe_router_score_function', 'sigmoid')
        if llm == 'deepseek_v32':
            res['experimental_attention_variant'] = 'dsa'
        elif llm == 'deepseek_v4':
            res.setdefault('v_head_dim', res.get('kv_channels'))
            res['experimental_attention_variant'] = 'dsv4_hybrid'
            res['moe_router_enable_expert_bias'] = True
            res['csa_window_size'] = window
            res['enable_hyper_connections'] = True
            ratios = res.pop('csa_compress_ratios', None) or {}
            res['csa_compress_ratios'] = [ratios.get(t, 0) for t in (layer_types or [])]
            res['moe_n_hash_layers'] = len([t for t in (hash_layers or []) if t == 'hash_moe'])
    elif llm == 'hunyuan':
        res['n_shared_experts'] = n_shared
        for key in ('moe_ffn_hidden_size', 'n_shared_experts', 'moe_router_topk'):
            val = res.get(key)
            if isinstance(val, list) and val and min(val) == max(val):
                res[key] = val[0]
        n_shared = res.pop('n_shared_experts')
    elif llm in {'ernie4_5', 'ernie4_5_moe', 'glm4'}:
        res['rotary_interleaved'] = True
        if llm == 'ernie4_5_moe':       # softmax probabilities plus a correction bias select the experts
            res['moe_router_enable_expert_bias'] = True
            res['moe_router_bias_update_rate'] = 0.0      # a checkpoint value, not moved by the balancing rule
        if llm == 'glm4':
            res['post_sublayer_layernorm'] = True
    elif hf_type in {'gemma4', 'gemma4_unified'} or llm == 'gemma4_text':
        res['qk_layernorm'] = True
        res['window_size'] = f'{window - 1},0'
        res['window_attn_skip_freq'] = _window_pattern(layer_types)
        res['softmax_scale'] = 1.
        res['swiglu'] = False
        res['gated_linear_unit'] = True
        res['activation_func'] = partial(F.gelu, approximate='tanh')
    elif llm == 'mistral':
        res['add_qkv_bias'] = False
    elif llm == 'gpt_oss':
        res.update(add_bias_linear=True, bias_dropout_fusion=False, softmax_type='learnable', swiglu=False,
                   quick_geglu=True, activation_func_clamp_value=7, glu_linear_offset=1)
        res['window_size'] = f'{window - 1},0'
        res['window_attn_skip_freq'] = '2' if layer_types is None else _window_pattern(layer_types)
    elif llm in {'glm4_moe', 'glm4_moe_lite', 'glm_moe_dsa'} or hf_type == 'glm4v_moe':
        res['moe_router_score_function'] = 'sigmoid'
        if llm in {'glm4_moe_lite', 'glm_moe_dsa'}:
            res['qk_layernorm'] = True
            res.pop('num_query_groups', None)
        if llm == 'glm_moe_dsa':
            res['experimental_attention_variant'] = 'dsa'
            res['mla_rope_interleaved'] = bool(res.pop('rotary_interleaved', False))
    elif llm == 'qwen3_next' or hf_type in {'qwen3_5', 'qwen3_5_moe'}:
        res['layernorm_zero_centered_gamma'] = True
        res['attention_output_gate'] = True
        if get_env_args('USE_MCORE_GDN', bool, True):
            res['experimental_attention_variant'] = 'gated_delta_net'
        res.setdefault('linear_attention_freq', 4)
    elif llm == 'minimax_m2':
        res['add_qkv_bias'] = False
        res['qk_layernorm_full'] = True
        # the architecture always routes with sigmoid scores plus a correction bias, whether or not the config
        # spells it out
        res.setdefault('moe_router_score_function', 'sigmoid')
        res['moe_router_enable_expert_bias'] = True
    elif llm == 'olmoe':
        res['qk_layernorm'] = True
        res['qk_layernorm_full'] = True
    elif hf_type == 'llama4':
        if res.pop('qk_layernorm', False):
            res['qk_l2_norm'] = True
        res.update(no_rope_freq=4, moe_apply_probs_on_input=True, rotary_interleaved=True,
                   moe_router_score_function='sigmoid', moe_router_enable_expert_bias=False)
        res['moe_ffn_hidden_size'] = res['ffn_hidden_size']
        res['ffn_hidden_size'] = mlp_ffn
        res['moe_shared_expert_intermediate_size'] = res['moe_ffn_hidden_size']
        if moe_step is not None and moe_step > 1:
            pat = ['1' if i % moe_step == (moe_step - 1) else '0' for i in range(res['num_layers'])]
            res['moe_layer_freq'] = '[' + ','.join(pat) + ']'
    elif hf_type == 'glm4v':
        res['rotary_interleaved'] = True
        res['post_sublayer_layernorm'] = True
    elif llm == 'bailing_hybrid':
        res.update(qk_layernorm=True, add_qkv_bias=False, moe_router_score_function='sigmoid',
                   moe_router_load_balancing_type='seq_aux_loss', experimental_attention_variant='lightning')
        # every `layer_group_size`-th layer and the tail that does not fill a group use full (MLA) attention
        group = getattr(hf_config, 'layer_group_size', None) if not isinstance(hf_config, dict) else \
            hf_config.get('layer_group_size')
        if group:
            n = res['num_layers']
            tail = n // group * group
            res['linear_attention_freq'] = [0 if ((i + 1) % group == 0 or i >= tail) else 1 for i in range(n)]

    if 'partial_rotary_factor' not in res and 'partial_rotary_factor' in rope_scaling:
        res['partial_rotary_factor'] = rope_scaling['partial_rotary_factor']
    if 'rotary_base' not in res and 'rope_theta' in rope_scaling:
        res['rotary_base'] = int(rope_scaling['rope_theta'])
    if rope_scaling.get('mrope_section') is not None:
        res['position_embedding_type'] = 'mrope'
        res['mrope_section'] = rope_scaling['mrope_section']
        res['mrope_interleaved'] = bool(rope_scaling.get('mrope_interleaved', False)
                                        or rope_scaling.get('interleaved', False))
    if rope_scaling and set(rope_scaling.keys()) <= {'rope_theta', 'rope_type', 'type', 'partial_rotary_factor',
                                                     'mrope_section', 'mrope_interleaved', 'interleaved'} \
            and rope_scaling.get('rope_type', rope_scaling.get('type', 'default')) == 'default':
        res.pop('rope_scaling', None)  # nothing to scale: a plain table

    if first_k_dense is None and isinstance(hash_layers, (list, tuple)) and set(hash_layers) <= {'dense', 'sparse'} \
            and res.get('num_moe_experts'):
        # newer configs list the MLP type of every layer instead of `first_k_dense_replace`
        res['moe_layer_freq'] = '[' + ','.join('1' if t == 'sparse' else '0' for t in hash_layers) + ']'
    if first_k_dense is not None:
        res['moe_layer_freq'] = f'[0]*{first_k_dense}+[1]*{res["num_layers"] - first_k_dense}'
    if res.get('moe_router_score_function', 'softmax') == 'sigmoid' and 'moe_router_enable_expert_bias' not in res:
        res['moe_router_enable_expert_bias'] = True
    if n_shared is not None and 'moe_shared_expert_intermediate_size' not in res:
        res['moe_shared_expert_intermediate_size'] = n_shared * res['moe_ffn_hidden_size']
    return res
