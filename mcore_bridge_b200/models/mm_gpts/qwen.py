"""Qwen2-VL / Qwen2.5-VL / Qwen2.5-Omni / Qwen3-VL(-MoE) / Qwen3-Omni / Qwen3.5 towers and bridges.

Parity: reference ``src/mcore_bridge/model/mm_gpts/qwen.py``, ``qwen3_vl.py``, ``qwen3_omni.py``, ``qwen3_5_gdn.py``.
"""
from __future__ import annotations

import torch

from ...bridge.gpt_bridge import GPTBridge, MultimodalGPTBridge
from ..constant import ModelType
from ..register import ModelMeta, register_model
from .base import HFProxy, HuggingFaceVit, scatter_embeds, shard_token_aligned


class Qwen2VLVit(HuggingFaceVit):
    module_mapping = {'model.visual': 'visual'}
    _vision_tower = ['visual']
    _aligner = ['visual.merger']

    def tower_class(self):
        from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel
        return Qwen2VisionTransformerPretrainedModel

    def prepare_model(self, hf_config):
        self.visual = self.tower_class()._from_config(hf_config.vision_config)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        return self.merge_media(inputs_embeds, inputs, self.visual, self.hf_config)


class Qwen2_5VLVit(Qwen2VLVit):

    def tower_class(self):
        from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
        return Qwen2_5_VisionTransformerPretrainedModel


class Qwen2VLBridge(MultimodalGPTBridge):
    # on disk the language model sits directly under ``model.``; the first releases also kept the tower at top level
    hf_state_dict_mapping = {
        'model.layers': 'model.language_model.layers',
        'model.embed_tokens': 'model.language_model.embed_tokens',
        'model.norm': 'model.language_model.norm',
    }
    hf_load_aliases = {'visual': 'model.visual'}


register_model(ModelMeta(ModelType.qwen2_vl, ['qwen2_vl'], bridge_cls=Qwen2VLBridge, visual_cls=Qwen2VLVit))
register_model(ModelMeta(ModelType.qwen2_5_vl, ['qwen2_5_vl'], bridge_cls=Qwen2VLBridge, visual_cls=Qwen2_5VLVit))


# ---------------------------------------------------------------------------------------------- Qwen3-VL (deepstack)
class Qwen3VLVit(HuggingFaceVit):
    module_mapping = {'model.visual': 'visual'}
    _vision_tower = ['visual']
    _aligner = ['visual.merger', 'visual.deepstack_merger_list']

    def prepare_model(self, hf_config):
        if self.config.hf_model_type == 'qwen3_vl_moe':
            from transformers.models.qwen3_vl_moe import Qwen3VLMoeVisionModel as VisionModel
        else:
            from transformers.models.qwen3_vl import Qwen3VLVisionModel as VisionModel
        self.visual = VisionModel._from_config(hf_config.vision_config)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        return self.merge_media_deepstack(inputs_embeds, inputs, self.visual, self.hf_config)

    def merge_media_deepstack(self, inputs_embeds, inputs, visual, hf_config):
        """Like ``merge_media`` and additionally returns the per-layer deepstack features restricted to this rank's
        tokens (context-parallel chunks, then the sequence-parallel slice)."""
        ids = inputs['input_ids']
        dummy = inputs.get('pixel_values') is None and inputs.get('pixel_values_videos') is None
        img, vid, deep, n_img = self.encode_media(visual, inputs, hf_config)
        deep = torch.stack(list(deep), 0)                                  # [L, n_media, H], tower order
        if dummy:
            return {'inputs_embeds': inputs_embeds + img.mean().to(inputs_embeds.dtype) * 0.0,
                    'visual_pos_masks': None, 'deepstack_visual_embeds': deep}
        inputs_embeds, m_img = scatter_embeds(inputs_embeds, ids, hf_config.image_token_id, img)
        inputs_embeds, m_vid = scatter_embeds(inputs_embeds, ids, hf_config.video_token_id, vid)
        m_img, m_vid = m_img.reshape(-1), m_vid.reshape(-1)
        if img is None:
            m_img = torch.zeros_like(m_img)
        if vid is None:
            m_vid = torch.zeros_like(m_vid)
        mask = m_img | m_vid
        if img is not None and vid is not None:
            # the tower saw [images | videos]; the stream interleaves them, so re-order into stream order
            joint = deep.new_zeros(deep.shape[0], int(mask.sum()), deep.shape[-1])
            joint[:, m_img[mask]] = deep[:, :n_img]
            joint[:, m_vid[mask]] = deep[:, n_img:]
            deep = joint
        cu = getattr(inputs.get('packed_seq_params'), 'cu_seqlens_q', None)
        b, s = ids.shape
        if b > 1 and self.config.context_parallel_size > 1:
            raise ValueError('deepstack with context parallelism expects one packed row per micro-batch')
        local_mask, local_deep = shard_token_aligned(mask, deep, cu, self.config)
        return {'inputs_embeds': inputs_embeds, 'visual_pos_masks': local_mask, 'deepstack_visual_embeds': local_deep}


class Qwen3VLMoeBridge(MultimodalGPTBridge):
    """Experts are stored fused (``experts.gate_up_proj`` / ``experts.down_proj``; input- or output-major depending on
    the Transformers release that wrote the checkpoint — reference
    ``src/mcore_bridge/bridge/gpt_bridge.py:765-773``)."""
    hf_fused_experts = True


register_model(ModelMeta(ModelType.qwen3_vl, ['qwen3_vl'], bridge_cls=MultimodalGPTBridge, visual_cls=Qwen3VLVit))
register_model(ModelMeta('qwen3_vl_moe', ['qwen3_vl_moe'], bridge_cls=Qwen3VLMoeBridge, visual_cls=Qwen3VLVit))


# ---------------------------------------------------------------------------------------------- audio helpers
class _AudioMixin:
    """Audio encoders of the Omni / ASR thinkers; the HF thinker class's ``get_audio_features`` is borrowed."""
    audio_token_attr = 'audio_token_id'

    def audio_embeds(self, input_features, feature_attention_mask):
        res = self.model_cls.get_audio_features(HFProxy(self, self.thinker_config), input_features,
                                                feature_attention_mask)
        return getattr(res, 'last_hidden_state', res)

    def merge_audio(self, inputs_embeds, inputs):
        ids = inputs['input_ids']
        feats, fmask = inputs.get('input_features'), inputs.get('feature_attention_mask')
        tower = self.audio_tower
        p = next(tower.parameters())
        if feats is None:       # keep the encoder in the graph on text-only batches
            feats = torch.zeros(1, 128, 128, dtype=p.dtype, device=p.device)
            fmask = torch.ones(1, 128, dtype=torch.bool, device=p.device)
            return inputs_embeds + self.audio_embeds(feats, fmask).mean().to(inputs_embeds.dtype) * 0.0
        emb = self.audio_embeds(feats.to(p.dtype), fmask)
        out, _ = scatter_embeds(inputs_embeds, ids, getattr(self.thinker_config, self.audio_token_attr), emb)
        return out


class _ThinkerBridge(GPTBridge):
    hf_layers_prefix = 'thinker.model.layers'
    hf_embed_key = 'thinker.model.embed_tokens.weight'
    hf_final_layernorm_key = 'thinker.model.norm.weight'
    hf_lm_head_key = 'thinker.lm_head.weight'
    hf_score_key = 'thinker.score.weight'


class Qwen2_5OmniVit(_AudioMixin, HuggingFaceVit):
    module_mapping = {'thinker.audio_tower': 'audio_tower', 'thinker.visual': 'visual'}
    _vision_tower = ['audio_tower', 'visual']
    _aligner = ['audio_tower.proj', 'visual.merger']
    _generator = ['talker', 'token2wav']
    audio_token_attr = 'audio_token_index'

    def prepare_model(self, hf_config):
        from transformers.models.qwen2_5_omni import modeling_qwen2_5_omni as m
        self.thinker_config = hf_config.thinker_config
        self.audio_tower = m.Qwen2_5OmniAudioEncoder._from_config(self.thinker_config.audio_config)
        self.visual = m.Qwen2_5OmniVisionEncoder._from_config(self.thinker_config.vision_config)
        self.model_cls = m.Qwen2_5OmniThinkerForConditionalGeneration

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        out = self.merge_media(inputs_embeds, inputs, self.visual, self.thinker_config)
        return self.merge_audio(out, inputs)


class Qwen3OmniVit(_AudioMixin, Qwen3VLVit):
    module_mapping = {'thinker.audio_tower': 'audio_tower', 'thinker.visual': 'visual'}
    _vision_tower = ['audio_tower', 'visual']
    _aligner = ['audio_tower.proj1', 'audio_tower.proj2', 'visual.merger', 'visual.merger_list']
    _generator = ['talker', 'code2wav']

    def prepare_model(self, hf_config):
        from transformers.models.qwen3_omni_moe import modeling_qwen3_omni_moe as m
        self.thinker_config = hf_config.thinker_config
        self.audio_tower = m.Qwen3OmniMoeAudioEncoder._from_config(self.thinker_config.audio_config)
        self.visual = m.Qwen3OmniMoeVisionEncoder._from_config(self.thinker_config.vision_config)
        self.model_cls = m.Qwen3OmniMoeThinkerForConditionalGeneration

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        res = self.merge_media_deepstack(inputs_embeds, inputs, self.visual, self.thinker_config)
        res['inputs_embeds'] = self.merge_audio(res['inputs_embeds'], inputs)
        return res


class Qwen3ASRVit(_AudioMixin, HuggingFaceVit):
    module_mapping = {'thinker.audio_tower': 'audio_tower'}
    _vision_tower = ['audio_tower']
    _aligner = ['audio_tower.proj1', 'audio_tower.proj2']
    test_mm_type = 'audio'

    def prepare_model(self, hf_config):
        # the ASR encoder ships in the separate ``qwen_asr`` package
        from qwen_asr.core.transformers_backend import modeling_qwen3_asr as m
        self.thinker_config = hf_config.thinker_config
        self.audio_tower = m.Qwen3ASRAudioEncoder._from_config(self.thinker_config.audio_config)
        self.model_cls = m.Qwen3ASRThinkerForConditionalGeneration

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        return self.merge_audio(inputs_embeds, inputs)


class Qwen3ASRBridge(_ThinkerBridge, MultimodalGPTBridge):
    hf_layers_prefix = 'thinker.model.layers'
    hf_embed_key = 'thinker.model.embed_tokens.weight'
    hf_final_layernorm_key = 'thinker.model.norm.weight'


register_model(ModelMeta(ModelType.qwen2_5_omni, ['qwen2_5_omni'], bridge_cls=_ThinkerBridge,
                         visual_cls=Qwen2_5OmniVit))
register_model(ModelMeta(ModelType.qwen3_omni, ['qwen3_omni_moe'], bridge_cls=_ThinkerBridge, visual_cls=Qwen3OmniVit))
register_model(ModelMeta(ModelType.qwen3_asr, ['qwen3_asr'], bridge_cls=Qwen3ASRBridge, visual_cls=Qwen3ASRVit))


# ---------------------------------------------------------------------------------------------- Qwen3.5 (GDN hybrid)
class Qwen3_5Vit(HuggingFaceVit):
    module_mapping = {'model.visual': 'visual'}
    _vision_tower = ['visual']
    _aligner = ['visual.merger']

    def prepare_model(self, hf_config):
        if self.config.hf_model_type == 'qwen3_5_moe':      # its vision config belongs to the MoE model's tower class
            from transformers.models.qwen3_5_moe import Qwen3_5MoeVisionModel as VisionModel
        else:
            from transformers.models.qwen3_5 import Qwen3_5VisionModel as VisionModel
        self.visual = VisionModel._from_config(hf_config.vision_config)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        return self.merge_media(inputs_embeds, inputs, self.visual, self.hf_config)


class Qwen3_5Bridge(MultimodalGPTBridge):
    split_gdn_projections = True     # in_proj_qkv / in_proj_z / in_proj_b / in_proj_a are separate tensors
    hf_fused_experts = True          # the MoE variant stores ``experts.gate_up_proj`` / ``experts.down_proj``


register_model(ModelMeta(ModelType.qwen3_5, ['qwen3_5', 'qwen3_5_moe'], bridge_cls=Qwen3_5Bridge,
                         visual_cls=Qwen3_5Vit))
