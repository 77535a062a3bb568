"""Multimodal wrapper: tiny Qwen3-VL (deepstack) and Qwen2.5-VL with an image in the prompt produce the same logits as
Transformers, and the tower's weights round-trip through the bridge key for key."""
import os

import pytest
import torch
from safetensors.torch import load_file

from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config


def _randomise(m):
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.02)
            elif 'bias' in n:
                p.normal_(0, 0.02)
            else:
                p.normal_(1.0, 0.1)
    return m


def _qwen3_vl():
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    c = Qwen3VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=512,
                         rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[8, 4, 4],
                                              mrope_interleaved=True), pad_token_id=0),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128,
                           num_position_embeddings=64, deepstack_visual_indexes=[0, 1]),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503,
        tie_word_embeddings=False)
    return c, Qwen3VLForConditionalGeneration(c)


def _qwen2_5_vl():
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    c = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                         rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[8, 4, 4]),
                         pad_token_id=0),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128, window_size=16,
                           fullatt_block_indexes=[1]),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503,
        tie_word_embeddings=False)
    return c, Qwen2_5_VLForConditionalGeneration(c)


def _qwen3_5():
    from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration
    c = Qwen3_5Config(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=512,
                         linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                         linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=4, pad_token_id=0,
                         rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[2, 1, 1],
                                              mrope_interleaved=True, partial_rotary_factor=0.25)),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128,
                           num_position_embeddings=64),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503,
        tie_word_embeddings=False)
    return c, Qwen3_5ForConditionalGeneration(c)


_TEXT = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, max_position_embeddings=512, pad_token_id=0, tie_word_embeddings=False)
_TOKENS = dict(image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503,
               tie_word_embeddings=False)


def _qwen2_vl():
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    c = Qwen2VLConfig(
        text_config=dict(_TEXT, rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[8, 4, 4])),
        vision_config=dict(depth=2, embed_dim=64, hidden_size=128, mlp_ratio=2, num_heads=4, in_channels=3,
                           patch_size=4, spatial_merge_size=2, temporal_patch_size=2), **_TOKENS)
    return c, Qwen2VLForConditionalGeneration(c)


def _qwen3_vl_moe():
    from transformers import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration
    c = Qwen3VLMoeConfig(
        text_config=dict(_TEXT, head_dim=32, moe_intermediate_size=64, num_experts=4, num_experts_per_tok=2,
                         decoder_sparse_step=1, mlp_only_layers=[],
                         rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[8, 4, 4],
                                              mrope_interleaved=True)),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128,
                           num_position_embeddings=64, deepstack_visual_indexes=[0]), **_TOKENS)
    return c, Qwen3VLMoeForConditionalGeneration(c)


def _glm4v():
    from transformers import Glm4vConfig, Glm4vForConditionalGeneration
    c = Glm4vConfig(
        text_config=dict(_TEXT, head_dim=32, rope_parameters=dict(rope_type='default', rope_theta=10000.0,
                                                                  mrope_section=[4, 6, 6], partial_rotary_factor=1.0)),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128, image_size=32),
        image_token_id=500, video_token_id=501, image_start_token_id=502, image_end_token_id=503,
        tie_word_embeddings=False)
    c.vision_start_token_id, c.vision_end_token_id = 502, 503        # names the shared input helper uses
    return c, Glm4vForConditionalGeneration(c)


def _qwen3_5_moe():
    from transformers import Qwen3_5MoeConfig, Qwen3_5MoeForConditionalGeneration
    c = Qwen3_5MoeConfig(
        text_config=dict(_TEXT, num_hidden_layers=4, head_dim=32, moe_intermediate_size=64,
                         shared_expert_intermediate_size=64, num_experts=4, num_experts_per_tok=2,
                         linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                         linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=4,
                         rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[2, 1, 1],
                                              mrope_interleaved=True, partial_rotary_factor=0.25)),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128,
                           num_position_embeddings=64), **_TOKENS)
    return c, Qwen3_5MoeForConditionalGeneration(c)


def _glm4v_moe():
    from transformers import Glm4vMoeConfig, Glm4vMoeForConditionalGeneration
    c = Glm4vMoeConfig(
        text_config=dict(_TEXT, head_dim=32, moe_intermediate_size=64, n_routed_experts=4, num_experts_per_tok=2,
                         n_shared_experts=1, first_k_dense_replace=1, n_group=1, topk_group=1,
                         rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[2, 3, 3],
                                              partial_rotary_factor=0.5)),
        vision_config=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128, image_size=32),
        image_token_id=500, video_token_id=501, image_start_token_id=502, image_end_token_id=503,
        tie_word_embeddings=False)
    c.vision_start_token_id, c.vision_end_token_id = 502, 503
    return c, Glm4vMoeForConditionalGeneration(c)


def _inputs(c):
    g = torch.Generator().manual_seed(0)
    grid = torch.tensor([[1, 8, 8]])                       # 64 patches -> 16 merged image tokens
    vc = c.vision_config
    feat = vc.in_channels * vc.temporal_patch_size * vc.patch_size ** 2
    pixels = torch.randn(64, feat, generator=g)
    ids = torch.randint(1, 400, (1, 48), generator=g)
    ids[0, 5] = c.vision_start_token_id
    ids[0, 6:22] = c.image_token_id
    ids[0, 22] = c.vision_end_token_id
    return ids, pixels, grid


@pytest.mark.parametrize('build', [_qwen3_vl, _qwen2_5_vl, _qwen3_5, _qwen2_vl, _qwen3_vl_moe, _glm4v, _glm4v_moe, _qwen3_5_moe])
def test_image_prompt_logits_and_roundtrip(build, tmp_path):
    torch.manual_seed(0)
    c, hf = build()
    hf = _randomise(hf.float().eval())
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    if build in (_qwen3_5, _qwen3_5_moe):
        # this Transformers version re-prefixes the language-model keys on save for this family; write the state
        # dict as it is in memory (the published layout) instead
        from safetensors.torch import save_file
        os.makedirs(d1)
        save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, os.path.join(d1, 'model.safetensors'))
        c.save_pretrained(d1)
    else:
        hf.save_pretrained(d1)
    ids, pixels, grid = _inputs(c)
    types = (ids == c.image_token_id).int()                # 0 text, 1 image
    kw = dict(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types)
    with torch.no_grad():
        out_hf = hf(**kw)
        pos, _ = hf.model.get_rope_index(ids, mm_token_type_ids=types, image_grid_thw=grid)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0].eval()
    assert model.visual is not None
    cfg.bridge.load_weights([model], d1)
    with torch.no_grad():
        out = model(ids, position_ids=pos, pixel_values=pixels, image_grid_thw=grid)
        text_only = model(ids.clamp(max=400), position_ids=pos)          # tower runs on a dummy grid, adds zero
    assert (out_hf.logits - out).abs().max().item() < 3e-5
    assert torch.isfinite(text_only).all()
    cfg.bridge.save_weights([model], d2)
    a, b = load_file(os.path.join(d1, 'model.safetensors')), load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(a) == sorted(b)
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_internvl_image_prompt_logits_and_roundtrip(tmp_path):
    """HF-native InternVL: ``pixel_values [n, 3, h, w]``, pixel-shuffle + projector borrowed from the Transformers class;
    the checkpoint uses the published key layout (``language_model.model.*``, ``vision_tower.*``)."""
    from safetensors.torch import save_file
    from transformers import InternVLConfig, InternVLForConditionalGeneration
    torch.manual_seed(0)
    c = InternVLConfig(
        text_config=dict(model_type='qwen2', vocab_size=512, hidden_size=128, intermediate_size=256,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, tie_word_embeddings=False),
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                           image_size=[32, 32], patch_size=[8, 8], num_channels=3),
        image_token_id=500, downsample_ratio=0.5, tie_word_embeddings=False)
    hf = _randomise(InternVLForConditionalGeneration(c).float().eval())
    renames = [('model.language_model.', 'language_model.model.'), ('lm_head.', 'language_model.lm_head.'),
               ('model.vision_tower.', 'vision_tower.'), ('model.multi_modal_projector.', 'multi_modal_projector.')]
    published = {}
    for k, v in hf.state_dict().items():
        for a, b in renames:
            if k.startswith(a):
                k = b + k[len(a):]
                break
        published[k] = v.contiguous()
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    os.makedirs(d1)
    save_file(published, os.path.join(d1, 'model.safetensors'))
    c.save_pretrained(d1)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(1, 400, (1, 32), generator=g)
    ids[0, 4:8] = 500                                      # 16 patches, pixel-shuffled to 4 image tokens
    pixels = torch.randn(1, 3, 32, 32, generator=g)
    with torch.no_grad():
        ref = hf(input_ids=ids, pixel_values=pixels).logits
    from transformers import AutoConfig
    cfg = ModelConfig(**hf_to_mcore_config(AutoConfig.from_pretrained(d1)), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0].eval()
    cfg.bridge.load_weights([model], d1)
    with torch.no_grad():
        assert (model(ids, pixel_values=pixels) - ref).abs().max().item() < 3e-5
    cfg.bridge.save_weights([model], d2)
    b = load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(b) == sorted(published)
    for k, v in published.items():
        assert torch.equal(b[k], v), k


def test_llama4_image_prompt_logits_and_roundtrip(tmp_path):
    """Llama-4: interleaved rope with a NoPE layer, weight-less RMS on q / k of the rotating layers, sigmoid top-1
    routing applied on the expert input, shared expert, fused expert tensors; vision tower through pixel shuffle."""
    from transformers import AutoConfig, Llama4Config, Llama4ForConditionalGeneration
    torch.manual_seed(0)
    c = Llama4Config(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=64, intermediate_size_mlp=256,
                         num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                         num_local_experts=4, num_experts_per_tok=1, interleave_moe_layer_step=1,
                         max_position_embeddings=512, tie_word_embeddings=False, attention_chunk_size=8192,
                         pad_token_id=0),
        vision_config=dict(hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                           image_size=32, patch_size=8, num_channels=3, vision_output_dim=64, projector_input_dim=64,
                           projector_output_dim=64, pixel_shuffle_ratio=0.5),
        image_token_index=500, boi_token_index=501, eoi_token_index=502, tie_word_embeddings=False)
    hf = _randomise(Llama4ForConditionalGeneration(c).float().eval())
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    hf.save_pretrained(d1)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(1, 400, (1, 32), generator=g)
    ids[0, 4:8] = 500
    pixels = torch.randn(1, 3, 32, 32, generator=g)
    with torch.no_grad():
        ref = hf(input_ids=ids, pixel_values=pixels).logits
    cfg = ModelConfig(**hf_to_mcore_config(AutoConfig.from_pretrained(d1)), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0].eval()
    cfg.bridge.load_weights([model], d1)
    with torch.no_grad():
        assert (model(ids, pixel_values=pixels) - ref).abs().max().item() < 3e-5
    cfg.bridge.save_weights([model], d2)
    a, b = load_file(os.path.join(d1, 'model.safetensors')), load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(a) == sorted(b)
    for k in a:
        assert torch.equal(a[k], b[k]), k
