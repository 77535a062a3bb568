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


# ---------------------------------------------------------------------------------------------- GPT-OSS
class GptOssBridge(GPTBridge):
    """Biased gate (``mlp.router.{weight,bias}``) and experts stored as fused, input-major tensors with gate and up
    columns interleaved: ``experts.gate_up_proj [E, H, 2F]`` (+ ``gate_up_proj_bias [E, 2F]``), ``experts.down_proj
    [E, F, H]`` (+ ``down_proj_bias [E, H]``).  Parity: reference ``src/mcore_bridge/bridge/gpt_bridge.py:696-700,
    894-900,1061-1088``."""

    def _ep_slice(self, t):
        from ...parallel import state as ps
        ep = ps.get_world_size('ep')
        if ep == 1:
            return t
        n, r = t.shape[0] // ep, ps.get_rank_in('ep')
        return t[r * n:(r + 1) * n]

    def _set_moe(self, mlp, hf_sd, prefix: str, to_mcore: bool):
        import torch
        router = mlp.router if mlp is not None else None
        self._direct(router, 'weight', hf_sd, prefix + 'router.weight', to_mcore)
        self._direct(router, 'bias', hf_sd, prefix + 'router.bias', to_mcore)
        ex = mlp.experts if mlp is not None else None
        ep_ = f'{prefix}{self.hf_experts_prefix}.'
        names = (('linear_fc1.weight', 'gate_up_proj'), ('linear_fc1.bias', 'gate_up_proj_bias'),
                 ('linear_fc2.weight', 'down_proj'), ('linear_fc2.bias', 'down_proj_bias'))
        for attr, key in names:
            mod, leaf = attr.split('.')
            param = getattr(getattr(ex, mod), leaf) if ex is not None else None
            fused_gate_up = key.startswith('gate_up')
            if to_mcore:
                if param is None:
                    continue
                t = self._ep_slice(self._load_hf(hf_sd, ep_ + key))
                if fused_gate_up:                                   # interleaved (gate, up) pairs -> [gate | up]
                    t = torch.cat([t[..., ::2], t[..., 1::2]], dim=-1)
                if leaf == 'weight':
                    t = t.transpose(1, 2)                           # input-major -> [E, out, in]
                with torch.no_grad():
                    param.copy_(t.to(device=param.device, dtype=param.dtype))
                continue
            if not self._agree(param is not None, self._device):
                continue
            t = None if param is None else param.detach()
            t = self._broadcast_pp(self._all_gather_ep(t), self._device)
            if t is None:
                continue
            if leaf == 'weight':
                t = t.transpose(1, 2)
            if fused_gate_up:
                g, u = t.chunk(2, dim=-1)
                t = torch.stack([g, u], dim=-1).reshape(*t.shape)   # back to interleaved pairs
            self._emit(hf_sd, ep_ + key, t.contiguous())


register_model(ModelMeta(ModelType.gpt_oss, ['gpt_oss'], bridge_cls=GptOssBridge))


# ---------------------------------------------------------------------------------------------- Ernie-4.5 MoE
class Ernie45MoeBridge(GPTBridge):
    """The selection bias lives in ``mlp.moe_statics.e_score_correction_bias`` with shape ``[1, E]``."""
    hf_expert_bias_key = 'moe_statics.e_score_correction_bias'
    hf_expert_bias_2d = True


register_model(ModelMeta('ernie4_5_moe', ['ernie4_5_moe'], bridge_cls=Ernie45MoeBridge))
