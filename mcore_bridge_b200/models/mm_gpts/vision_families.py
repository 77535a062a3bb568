"""GLM-4V(-MoE), InternVL (remote-code and HF-native), Kimi-VL / Kimi-K2.5, Llama-4, LLaVA-OneVision-1.5, Ovis2.5.

Towers whose modelling code is not part of ``transformers`` are fetched from the checkpoint directory with
``get_class_from_dynamic_module`` (``trust_remote_code`` style) when the tower is built.
Parity: reference ``src/mcore_bridge/model/mm_gpts/{glm,internvl,kimi_vl,llama4,llava,qwen}.py``.
"""
from __future__ import annotations

import torch
from torch import nn

from ...bridge.gpt_bridge import GPTBridge, MultimodalGPTBridge
from ..constant import ModelType
from ..register import ModelMeta, register_model
from .base import HFProxy, HuggingFaceVit, scatter_embeds


def _remote(name: str, hf_config):
    from transformers.dynamic_module_utils import get_class_from_dynamic_module
    return get_class_from_dynamic_module(name, hf_config.name_or_path)


def _param_of(module: nn.Module) -> torch.Tensor:
    return next(module.parameters())


class _NestedLMBridge(GPTBridge):
    """Checkpoints that keep a complete causal LM under ``language_model``."""
    hf_layers_prefix = 'language_model.model.layers'
    hf_embed_key = 'language_model.model.embed_tokens.weight'
    hf_final_layernorm_key = 'language_model.model.norm.weight'
    hf_lm_head_key = 'language_model.lm_head.weight'
    hf_score_key = 'language_model.score.weight'


# ---------------------------------------------------------------------------------------------- GLM-4V
class Glm4vVit(HuggingFaceVit):
    module_mapping = {'model.visual': 'visual'}
    _vision_tower = ['visual']
    _aligner = ['visual.merger']

    def prepare_model(self, hf_config):
        from transformers.models.glm4v_moe import Glm4vMoeVisionModel
        self.visual = Glm4vMoeVisionModel._from_config(hf_config.vision_config)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        return self.merge_media(inputs_embeds, inputs, self.visual, self.hf_config)


register_model(ModelMeta(ModelType.glm4v_moe, ['glm4v_moe'], bridge_cls=MultimodalGPTBridge, visual_cls=Glm4vVit))


def _register_glm4v():
    from ..gpts.families import Glm4Bridge

    class Glm4vBridge(Glm4Bridge, MultimodalGPTBridge):
        hf_layers_prefix = MultimodalGPTBridge.hf_layers_prefix
        hf_embed_key = MultimodalGPTBridge.hf_embed_key
        hf_final_layernorm_key = MultimodalGPTBridge.hf_final_layernorm_key

    register_model(ModelMeta(ModelType.glm4v, ['glm4v'], bridge_cls=Glm4vBridge, visual_cls=Glm4vVit))


_register_glm4v()


# ---------------------------------------------------------------------------------------------- InternVL
class _PixelTower(HuggingFaceVit):
    """Towers fed with ``pixel_values [n, 3, h, w]`` and one placeholder token id."""
    dummy_hw = 32

    def image_features(self, pixel_values) -> torch.Tensor:
        raise NotImplementedError

    def image_token_id(self, inputs) -> int:
        return self.hf_config.image_token_id

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        pv = inputs.get('pixel_values')
        p = _param_of(self)
        if pv is None:
            pv0 = torch.zeros(1, 3, self.dummy_hw, self.dummy_hw, dtype=p.dtype, device=p.device)
            return inputs_embeds + self.image_features(pv0).mean().to(inputs_embeds.dtype) * 0.0
        feats = self.image_features(pv.to(device=p.device, dtype=p.dtype))
        feats = feats.reshape(-1, feats.shape[-1])
        out, _ = scatter_embeds(inputs_embeds, inputs['input_ids'], self.image_token_id(inputs), feats)
        return out


class InternvlVit(_PixelTower):
    """InternVL-Chat (remote code): InternViT + pixel-shuffle + 2-layer MLP projector."""
    module_mapping = {'vision_model': 'vision_model', 'mlp1': 'mlp1'}
    _vision_tower = ['vision_model']
    _aligner = ['mlp1']

    def prepare_attn_impl(self):
        impl = getattr(self.config, 'vit_attn_impl', None) or 'flash_attention_2'
        self.hf_config.vision_config.use_flash_attn = 'flash' in impl and torch.cuda.is_available()

    def prepare_model(self, hf_config):
        if self.config.llm_model_type not in ('qwen2', 'qwen3', 'qwen3_moe', 'gpt_oss'):
            raise ValueError(f'{self.config.llm_model_type} is not supported for internvl_chat')
        vit_cls = _remote('modeling_internvl_chat.InternVisionModel', hf_config)
        self.model_cls = _remote('modeling_internvl_chat.InternVLChatModel', hf_config)
        self.vision_model = vit_cls._from_config(hf_config.vision_config)
        k = int(1 / hf_config.downsample_ratio) ** 2
        vh, lh = hf_config.vision_config.hidden_size, hf_config.llm_config.hidden_size
        self.mlp1 = nn.Sequential(nn.LayerNorm(vh * k), nn.Linear(vh * k, lh), nn.GELU(), nn.Linear(lh, lh)).to(
            _param_of(self.vision_model).dtype)
        self.select_layer, self.downsample_ratio = hf_config.select_layer, hf_config.downsample_ratio
        self.ps_version = hf_config.ps_version
        self._context_id = None

    def image_token_id(self, inputs):
        if self._context_id is None:
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(self.hf_config.name_or_path, trust_remote_code=True)
            self._context_id = tok.encode('<IMG_CONTEXT>', add_special_tokens=False)[0]
        return self._context_id

    def image_features(self, pixel_values):
        return self.model_cls.extract_feature(HFProxy(self, self.hf_config), pixel_values)


class InternvlBridge(_NestedLMBridge):
    pass


register_model(ModelMeta(ModelType.internvl_chat, ['internvl_chat'], bridge_cls=InternvlBridge, visual_cls=InternvlVit))


class InternvlHfVit(_PixelTower):
    module_mapping = {'model.vision_tower': 'vision_tower', 'model.multi_modal_projector': 'multi_modal_projector'}
    _vision_tower = ['vision_tower']
    _aligner = ['multi_modal_projector']

    def prepare_model(self, hf_config):
        from transformers import AutoModel
        from transformers.models.internvl.modeling_internvl import InternVLModel, InternVLMultiModalProjector
        self.vision_tower = AutoModel.from_config(hf_config.vision_config)
        self.multi_modal_projector = InternVLMultiModalProjector(hf_config).to(_param_of(self.vision_tower).dtype)
        self.model_cls = InternVLModel

    def image_features(self, pixel_values):
        c = self.hf_config
        res = self.model_cls.get_image_features(HFProxy(self, c), pixel_values,
                                                vision_feature_layer=c.vision_feature_layer,
                                                vision_feature_select_strategy=c.vision_feature_select_strategy)
        return getattr(res, 'pooler_output', res)


class InternvlHfBridge(MultimodalGPTBridge):
    hf_state_dict_mapping = {
        'language_model.lm_head': 'lm_head',
        'language_model.model': 'model.language_model',
        'vision_tower': 'model.vision_tower',
        'multi_modal_projector': 'model.multi_modal_projector',
    }


register_model(ModelMeta(ModelType.internvl, ['internvl'], bridge_cls=InternvlHfBridge, visual_cls=InternvlHfVit))


# ---------------------------------------------------------------------------------------------- Kimi
class KimiVLBridge(_NestedLMBridge):
    pass


class KimiVLVit(HuggingFaceVit):
    module_mapping = {'vision_tower': 'vision_tower', 'multi_modal_projector': 'multi_modal_projector'}
    _vision_tower = ['vision_tower']
    _aligner = ['multi_modal_projector']

    def prepare_model(self, hf_config):
        self.vision_tower = _remote('modeling_kimi_vl.MoonVitPretrainedModel', hf_config)._from_config(
            hf_config.vision_config)
        self.multi_modal_projector = _remote('modeling_kimi_vl.KimiVLMultiModalProjector', hf_config)(hf_config).to(
            _param_of(self.vision_tower).dtype)
        self.model_cls = _remote('modeling_kimi_vl.KimiVLForConditionalGeneration', hf_config)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        ids, pv = inputs['input_ids'], inputs.get('pixel_values')
        p = _param_of(self.vision_tower)
        proxy = HFProxy(self, self.hf_config)
        if pv is None or pv.shape[0] == 0:
            ps_ = self.hf_config.vision_config.patch_size
            pv0 = torch.zeros(16, 3, ps_, ps_, dtype=p.dtype, device=p.device)
            feats = self.model_cls._extract_image_features(proxy, pv0, torch.tensor([[4, 4]], device=p.device))
            feats = torch.cat(list(feats), 0) if isinstance(feats, (list, tuple)) else feats
            return inputs_embeds + feats.mean().to(inputs_embeds.dtype) * 0.0
        feats = self.model_cls._extract_image_features(proxy, pv.to(p.dtype), inputs['image_grid_hws'])
        return self.model_cls._merge_with_image_features(proxy, inputs_embeds.clone(), ids, feats)


class KimiK25Vit(HuggingFaceVit):
    module_mapping = {'vision_tower': 'vision_tower', 'mm_projector': 'mm_projector'}
    _vision_tower = ['vision_tower']
    _aligner = ['mm_projector']

    def prepare_model(self, hf_config):
        vit_cls, merger_cls, vit_cfg_cls, proj_cfg_cls = (_remote(f'modeling_kimi_k25.{n}', hf_config) for n in (
            'MoonViT3dPretrainedModel', 'PatchMergerMLP', 'VisionTowerConfig', 'ProjectorConfig'))
        if hf_config.vision_config.mm_projector_type != 'patchmerger':
            raise ValueError('only the patch-merger projector is supported')
        vit_cfg, proj_cfg = vit_cfg_cls(hf_config.vision_config), proj_cfg_cls(hf_config.vision_config)
        vit_cfg.torch_dtype = hf_config.torch_dtype
        self.vision_tower = vit_cls._from_config(vit_cfg)
        self.mm_projector = merger_cls(proj_cfg).to(hf_config.torch_dtype)
        self.model_cls = _remote('modeling_kimi_k25.KimiK25ForConditionalGeneration', hf_config)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        pv = inputs.get('pixel_values')
        if pv is None or pv.shape[0] == 0:
            return inputs_embeds
        p = _param_of(self.vision_tower)
        feats = self.model_cls._extract_image_features(HFProxy(self, self.hf_config), pv.to(p.dtype),
                                                       inputs['grid_thws'])
        feats = torch.cat(list(self.mm_projector(feats)), 0)
        out, _ = scatter_embeds(inputs_embeds, inputs['input_ids'], self.hf_config.media_placeholder_token_id, feats)
        return out


register_model(ModelMeta(ModelType.kimi_vl, ['kimi_vl'], bridge_cls=KimiVLBridge, visual_cls=KimiVLVit))
register_model(ModelMeta(ModelType.kimi_k25, ['kimi_k25'], bridge_cls=KimiVLBridge, visual_cls=KimiK25Vit))


# ---------------------------------------------------------------------------------------------- Llama-4
class Llama4Vit(_PixelTower):
    module_mapping = {'multi_modal_projector': 'multi_modal_projector', 'vision_model': 'vision_model'}
    _vision_tower = ['vision_model']
    _aligner = ['multi_modal_projector']
    dummy_hw = 336

    def prepare_model(self, hf_config):
        from transformers.models.llama4 import modeling_llama4 as m
        self.vision_model = m.Llama4VisionModel._from_config(hf_config.vision_config)
        self.multi_modal_projector = m.Llama4MultiModalProjector(hf_config).to(_param_of(self.vision_model).dtype)
        self.model_cls = m.Llama4ForConditionalGeneration

    def image_token_id(self, inputs):
        c = self.hf_config
        return getattr(c, 'image_token_id', None) or c.image_token_index

    def image_features(self, pixel_values):
        strategy = self.hf_config.vision_config.vision_feature_select_strategy
        res = self.model_cls.get_image_features(HFProxy(self, self.hf_config), pixel_values=pixel_values,
                                                vision_feature_select_strategy=strategy)
        res = getattr(res, 'last_hidden_state', res)
        return self.multi_modal_projector(res.reshape(-1, res.shape[-1]))


class Llama4Bridge(_NestedLMBridge):
    hf_mlp_prefix = 'feed_forward'
    hf_gate_key = 'router.weight'
    hf_shared_expert_prefix = 'shared_expert'
    hf_fused_experts = True


register_model(ModelMeta(ModelType.llama4, ['llama4'], bridge_cls=Llama4Bridge, visual_cls=Llama4Vit))


# ---------------------------------------------------------------------------------------------- LLaVA-OneVision-1.5
class LlavaOneVision1_5Vit(HuggingFaceVit):
    module_mapping = {'visual': 'visual'}
    _vision_tower = ['visual']
    _aligner = ['visual.merger']

    def prepare_model(self, hf_config):
        cls = _remote('modeling_llavaonevision1_5.RiceTransformerPretrainedModel', hf_config)
        self.visual = cls._from_config(hf_config.vision_config)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        return self.merge_media(inputs_embeds, inputs, self.visual, self.hf_config)


register_model(ModelMeta(ModelType.llava_onevision1_5, ['llava_onevision1_5'], visual_cls=LlavaOneVision1_5Vit))


# ---------------------------------------------------------------------------------------------- Ovis2.5
class Ovis2_5Bridge(GPTBridge):
    hf_layers_prefix = 'llm.model.layers'
    hf_embed_key = 'llm.model.embed_tokens.weight'
    hf_final_layernorm_key = 'llm.model.norm.weight'
    hf_lm_head_key = 'llm.lm_head.weight'
    hf_score_key = 'llm.score.weight'


class Ovis2_5Vit(HuggingFaceVit):
    """Ovis tokenises images into a soft distribution over a visual vocabulary (``visual_tokenizer``) and embeds it
    with ``vte``; negative token ids mark the image atoms (-300) and four indicator tokens (-301..-304)."""
    module_mapping = {'visual_tokenizer': 'visual_tokenizer', 'vte': 'vte'}
    _vision_tower = ['visual_tokenizer.vit', 'vte']
    _aligner = ['visual_tokenizer.head']
    ATOM_ID = -300
    INDICATOR_IDS = (-301, -302, -303, -304)

    def prepare_model(self, hf_config):
        from transformers import AutoModel

        from ...utils.env import get_env_args
        self.min_pixels = get_env_args('min_pixels', int, 448 * 448)
        self.max_pixels = get_env_args('max_pixels', int, 1344 * 1792)
        emb_cls = _remote('modeling_ovis2_5.VisualEmbedding', hf_config)
        tok_cls = _remote('modeling_ovis2_5.VisualTokenizer', hf_config)
        vit = AutoModel.from_config(hf_config.vit_config)
        dt = _param_of(vit).dtype
        self.visual_tokenizer = tok_cls(vit=vit, visual_vocab_size=hf_config.visual_vocab_size,
                                        image_processor_name_or_path=hf_config.name_or_path)
        self.visual_tokenizer.head.to(dtype=dt)
        self.vte = emb_cls(hf_config.visual_vocab_size, hf_config.hidden_size, dtype=dt)
        n = len(self.INDICATOR_IDS)
        self.register_buffer('indicator_index', torch.arange(hf_config.visual_vocab_size - n,
                                                             hf_config.visual_vocab_size), persistent=False)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        ids = inputs['input_ids']
        marks = self.vte(self.indicator_index.to(inputs_embeds.device)).to(inputs_embeds.dtype)
        out = inputs_embeds
        for i, tid in enumerate(self.INDICATOR_IDS):
            n = int((ids == tid).sum())
            if n:
                out, _ = scatter_embeds(out, ids, tid, marks[i].expand(n, -1))
        pv, grids = inputs.get('pixel_values'), inputs.get('grid_thws')
        if pv is None:
            from PIL import Image
            pv, grids = self.visual_tokenizer.preprocess(Image.new('RGB', (32, 32), (0, 0, 0)),
                                                         min_pixels=self.min_pixels, max_pixels=self.max_pixels)
            emb = self.vte(self.visual_tokenizer(pv.to(out.device), grids.to(out.device)))
            return out + emb.mean().to(out.dtype) * 0.0
        emb = self.vte(self.visual_tokenizer(pv, grids))
        out, _ = scatter_embeds(out, ids, self.ATOM_ID, emb)
        return out


register_model(ModelMeta(ModelType.ovis2_5, ['ovis2_5'], bridge_cls=Ovis2_5Bridge, visual_cls=Ovis2_5Vit))
