"""Text families that differ from the generic decoder only in a few modules or checkpoint key names.

The model-side differences are config switches resolved by the parser (``post_sublayer_layernorm`` for GLM-4's
sandwich norms, ``qk_layernorm_full`` for the all-channel q/k norm of OLMoE and MiniMax-M2), so each family here is a
bridge subclass naming its checkpoint layout.  Parity: reference ``src/mcore_bridge/model/gpts/{glm4,olmoe,
minimax_m2,hunyuan,bailing_moe,qwen3_emb}.py``.
"""
from ...bridge.gpt_bridge import GPTBridge
from ..constant import ModelType
from ..register import ModelMeta, register_model


class Glm4Bridge(GPTBridge):
    """GLM-4 dense: sandwich norms (``post_self_attn_layernorm`` / ``post_mlp_layernorm``), fused ``gate_up_proj``."""
    hf_fused_gate_up = True


class OLMoEBridge(GPTBridge):
    """OLMoE: ``q_norm`` / ``k_norm`` span all heads (weights ``[n_heads * d]``, sharded by head)."""


class MinimaxM2Bridge(GPTBridge):
    hf_mlp_prefix = 'block_sparse_moe'
    hf_expert_bias_key = 'e_score_correction_bias'
    hf_expert_proj_names = ('w1', 'w3', 'w2')


class HyV3Bridge(GPTBridge):
    hf_gate_key = 'router.gate.weight'
    hf_expert_bias_key = 'expert_bias'
    hf_shared_expert_prefix = 'shared_mlp'


class BailingMoeBridge(GPTBridge):
    """Ling / Ring (bailing_moe): fused ``query_key_value`` stored ``[all q | all k | all v]``, ``dense`` output
    projection, ``word_embeddings``."""
    hf_embed_key = 'model.word_embeddings.weight'
    hf_attn_prefix = 'attention'
    hf_q_norm_key = 'query_layernorm.weight'
    hf_k_norm_key = 'key_layernorm.weight'
    hf_expert_bias_key = 'gate.expert_bias'
    hf_o_proj_key = 'dense.weight'
    hf_fused_qkv_key = 'query_key_value'
    hf_mtp_final_layernorm_key = 'final_layernorm.weight'


class BailingHybridBridge(BailingMoeBridge):
    """Ling-2.5 / Ring-linear: groups of lightning-attention layers closed by an MLA layer."""


class Qwen3EmbBridge(GPTBridge):
    """Qwen3-Embedding checkpoints are a bare ``Qwen3Model``: keys lack the ``model.`` prefix."""
    hf_layers_prefix = 'layers'
    hf_embed_key = 'embed_tokens.weight'
    hf_final_layernorm_key = 'norm.weight'


register_model(ModelMeta(ModelType.glm4, ['glm4'], bridge_cls=Glm4Bridge))
register_model(ModelMeta(ModelType.olmoe, ['olmoe'], bridge_cls=OLMoEBridge))
register_model(ModelMeta(ModelType.minimax_m2, ['minimax_m2'], bridge_cls=MinimaxM2Bridge))
register_model(ModelMeta(ModelType.hy_v3, ['hy_v3'], bridge_cls=HyV3Bridge))
register_model(ModelMeta(ModelType.bailing_moe, ['bailing_moe'], bridge_cls=BailingMoeBridge))
register_model(ModelMeta(ModelType.bailing_hybrid, ['bailing_hybrid'], bridge_cls=BailingHybridBridge))
register_model(ModelMeta(ModelType.qwen3_emb, [], bridge_cls=Qwen3EmbBridge))
