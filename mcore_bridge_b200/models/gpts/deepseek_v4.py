"""DeepSeek-V4: hyper-connection residual streams, hash-routed first MoE layers, one shared key / value head with a
grouped low-rank output projection (``layers/dsv4_attention.py``).

Available: every layer whose ``layer_types`` entry is ``sliding_attention`` (compression ratio 0).  Layers with
compressed key / value blocks are refused by ``ModelConfig`` — the reference builds them from a Megatron-Core
development branch (``src/mcore_bridge/model/gpts/deepseek_v4.py:17-29,364-372``), so their definition is not in its
source tree.

Checkpoint layout (reference ``:375-509``): keys carry no ``model.`` prefix on disk, quantisation scales are stored as
``<name>.scale``, linears of the feed-forward blocks are called ``w1`` / ``w3`` / ``w2``, attention projections
``wq_a`` / ``wq_b`` / ``wkv`` / ``wo_a`` / ``wo_b``, norms ``attn_norm`` / ``ffn_norm`` / ``q_norm`` / ``kv_norm``,
the per-head sink ``attn_sink``; expert weights may be fp4 (two e2m1 values per byte, low nibble first) or fp8 with
block scales and are dequantised on load.
"""
from __future__ import annotations

import torch

from ...bridge.gpt_bridge import GPTBridge
from ...utils.dequantizer import Fp8Dequantizer, fp4_e2m1_to_float
from ..constant import ModelType
from ..gpt_model import GPTModel
from ..register import ModelLoader, ModelMeta, register_model
from ..rope import RotaryEmbedding

_FFN_NAMES = (('.w1.', '.gate_proj.'), ('.w3.', '.up_proj.'), ('.w2.', '.down_proj.'))


class DeepseekV4GPTModel(GPTModel):
    """``rope_scaling`` of this family holds one entry per layer kind (``main`` for sliding-window layers,
    ``compress`` for compressed ones: reference ``:345-360``); the table the layers read is the ``main`` one."""

    def __init__(self, config, *args, **kwargs):
        super().__init__(config, *args, **kwargs)
        rs = config.rope_scaling or {}
        if 'main' in rs or 'compress' in rs:
            self.rotary_pos_emb = RotaryEmbedding(config, rope_scaling_override=rs.get('main') or None)
        if self.rotary_pos_emb is not None and abs(self.rotary_pos_emb.attention_scaling - 1.0) > 1e-6:
            # the attention output is rotated back with the same table: the rotation has to be a pure one
            raise NotImplementedError('DeepSeek-V4 sliding-window layers: a rotary table with an attention scaling '
                                      f'factor ({self.rotary_pos_emb.attention_scaling}) is not supported')


class DeepseekV4Loader(ModelLoader):
    model_cls = DeepseekV4GPTModel


class DeepseekV4Bridge(GPTBridge):
    hf_embed_key = 'model.embed.weight'
    hf_lm_head_key = 'model.head.weight'
    hf_score_key = 'model.score.weight'
    hf_attn_prefix = 'attn'
    hf_mlp_prefix = 'ffn'
    hf_input_layernorm_key = 'attn_norm.weight'
    hf_post_attention_layernorm_key = 'ffn_norm.weight'
    hf_expert_bias_key = 'gate.bias'
    hf_shared_expert_prefix = 'shared_experts'
    # non-empty so that load and export pass every key through ``_modernise_key`` / ``_legacy_key`` below
    hf_state_dict_mapping = {'layers': 'model.layers'}

    # ------------------------------------------------------------------ key names: disk <-> internal
    def _modernise_key(self, key: str) -> str:
        if not key.startswith('model.'):
            key = 'model.' + key
        if key.endswith('.scale'):
            key = key[:-len('.scale')] + '.weight_scale_inv'
        for disk, internal in _FFN_NAMES:
            key = key.replace(disk, internal)
        return key

    def _legacy_key(self, key: str) -> str:
        if key.startswith('model.'):
            key = key[len('model.'):]
        if key.endswith('.weight_scale_inv'):
            key = key[:-len('.weight_scale_inv')] + '.scale'
        for disk, internal in _FFN_NAMES:
            key = key.replace(internal, disk)
        return key

    def _peft_key(self, key: str, to_mcore: bool) -> str:
        pre = 'base_model.model.'
        if not key.startswith(pre):
            return key
        inner = key[len(pre):]
        return pre + (self._modernise_key(inner) if to_mcore else self._legacy_key(inner))

    def _peft_module_name(self, name: str) -> str:
        return {'gate_proj': 'w1', 'up_proj': 'w3', 'down_proj': 'w2'}.get(name, name)

    # ------------------------------------------------------------------ fp4 tensors
    def _load_hf(self, hf_sd, key: str) -> torch.Tensor:
        t = hf_sd[key].load()
        sk = key + '_scale_inv'
        if sk in hf_sd and t.dtype == torch.int8:
            # packed e2m1 pairs [rows, cols / 2] with one scale per block of the unpacked row; the block sizes are read
            # off the scale grid (reference ``:499-509``)
            scale = hf_sd[sk].load()
            return Fp8Dequantizer().convert(fp4_e2m1_to_float(t), scale.reshape(-1, scale.shape[-1]))
        return super()._load_hf(hf_sd, key)

    # ------------------------------------------------------------------ attention
    def _set_layer_attn(self, layer, hf_sd, prefix: str, to_mcore: bool):
        attn = layer.self_attention if layer is not None else None
        ap = f'{prefix}{self.hf_attn_prefix}.'
        self._direct(layer, 'input_layernorm.weight', hf_sd, prefix + self.hf_input_layernorm_key, to_mcore)
        self._direct(attn, 'linear_q_down_proj.weight', hf_sd, ap + 'wq_a.weight', to_mcore)
        self._direct(attn, 'q_layernorm.weight', hf_sd, ap + 'q_norm.weight', to_mcore)
        self._direct(attn, 'linear_q_up_proj.weight', hf_sd, ap + 'wq_b.weight', to_mcore, tp_dim=0)
        self._direct(attn, 'linear_kv_proj.weight', hf_sd, ap + 'wkv.weight', to_mcore)
        self._direct(attn, 'kv_layernorm.weight', hf_sd, ap + 'kv_norm.weight', to_mcore)
        self._direct(attn, 'core_attention.attn_sink', hf_sd, ap + 'attn_sink', to_mcore, tp_dim=0)
        self._direct(attn, 'linear_o_group_proj', hf_sd, ap + 'wo_a.weight', to_mcore, tp_dim=0)
        self._direct(attn, 'linear_proj.weight', hf_sd, ap + 'wo_b.weight', to_mcore, tp_dim=1)

    # ------------------------------------------------------------------ MoE: hash-routed layers have no selection bias
    def _set_moe(self, mlp, hf_sd, prefix: str, to_mcore: bool):
        cfg = self.config
        router = mlp.router if mlp is not None else None
        hashed = self._agree(bool(router is not None and getattr(router, 'is_hash_layer', False)), self._device)
        keep = cfg.moe_router_enable_expert_bias
        if hashed:
            cfg.moe_router_enable_expert_bias = False
        try:
            super()._set_moe(mlp, hf_sd, prefix, to_mcore)
        finally:
            cfg.moe_router_enable_expert_bias = keep


register_model(ModelMeta(ModelType.deepseek_v4, ['deepseek_v4'], bridge_cls=DeepseekV4Bridge, loader=DeepseekV4Loader))
