"""Inverse frequencies and attention scaling of every RoPE scaling family against Transformers'
``ROPE_INIT_FUNCTIONS``; MRoPE tables against the Qwen3-VL rotary module."""
import pytest
import torch

from mcore_bridge_b200.models.rope import compute_inv_freq


def _hf(rope_type, params, dim=64, base=10000.0, max_pos=4096, seq_len=None):
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    rp = dict(rope_type=rope_type, rope_theta=base, **params)
    c = LlamaConfig(hidden_size=dim * 4, num_attention_heads=4, head_dim=dim, max_position_embeddings=max_pos,
                    rope_parameters=rp)
    fn = ROPE_INIT_FUNCTIONS[rope_type]
    return fn(c, 'cpu', seq_len=seq_len) if rope_type == 'dynamic' else fn(c, 'cpu')


CASES = [
    ('linear', dict(factor=4.0), None),
    ('dynamic', dict(factor=2.0), 8192),
    ('yarn', dict(factor=8.0, original_max_position_embeddings=512), None),
    ('yarn', dict(factor=40.0, original_max_position_embeddings=128, mscale=1.0, mscale_all_dim=0.707,
                  beta_fast=32, beta_slow=1), None),
    ('llama3', dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=1024), None),
    ('longrope', dict(factor=4.0, short_factor=[1.0 + 0.01 * i for i in range(32)],
                      long_factor=[2.0 + 0.05 * i for i in range(32)], original_max_position_embeddings=4096), None),
]


@pytest.mark.parametrize('rope_type,params,seq_len', CASES)
def test_inv_freq_matches_transformers(rope_type, params, seq_len):
    dim, base, max_pos = 64, 10000.0, 4096
    ref_inv, ref_scale = _hf(rope_type, params, dim, base, max_pos, seq_len)
    rs = dict(rope_type=rope_type, **params)
    inv, scale = compute_inv_freq(rope_type, base, dim, rs, max_pos, seq_len=seq_len)
    assert torch.allclose(inv, ref_inv.float(), rtol=1e-6, atol=0), (inv - ref_inv).abs().max()
    assert abs(scale - float(ref_scale)) < 1e-6


def test_default_and_dynamic_alpha():
    inv, scale = compute_inv_freq('default', 1e6, 128, None, 4096)
    ref = 1.0 / (1e6 ** (torch.arange(0, 128, 2).float() / 128))
    assert torch.allclose(inv, ref) and scale == 1.0
    # Hunyuan's NTK-alpha: base * alpha ** (dim / (dim - 2))
    inv2, _ = compute_inv_freq('dynamic_alpha', 10000.0, 128, dict(alpha=1000.0), 4096)
    nb = 10000.0 * 1000.0 ** (128 / 126)
    assert torch.allclose(inv2, 1.0 / (nb ** (torch.arange(0, 128, 2).float() / 128)))


def test_mrope_tables_match_qwen3_vl():
    from transformers import Qwen3VLConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLTextRotaryEmbedding

    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    from mcore_bridge_b200.models.rope import RotaryEmbedding
    full = Qwen3VLConfig(
        text_config=dict(vocab_size=64, hidden_size=128, intermediate_size=64, num_hidden_layers=1,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=512,
                         rope_parameters=dict(rope_type='default', rope_theta=10000.0, mrope_section=[8, 4, 4],
                                              mrope_interleaved=True)),
        vision_config=dict(depth=1, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4,
                           out_hidden_size=128, num_position_embeddings=16, deepstack_visual_indexes=[0]))
    tc = full.text_config
    hf_rot = Qwen3VLTextRotaryEmbedding(tc)
    pos = torch.stack([torch.arange(24), torch.arange(24) // 2, torch.arange(24) % 5]).unsqueeze(1)   # [3, 1, 24]
    cos_ref, sin_ref = hf_rot(torch.zeros(1, 24, 128), pos)
    cfg = ModelConfig(**hf_to_mcore_config(full), params_dtype=torch.float32)
    cos, sin = RotaryEmbedding(cfg)(pos.reshape(3, -1))
    half = cos.shape[-1]
    assert torch.allclose(cos, cos_ref[0, :, :half], atol=1e-6) and torch.allclose(sin, sin_ref[0, :, :half], atol=1e-6)
