import pytest
import torch

from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
from mcore_bridge_b200.config.model_config import _eval_pattern, tuple_type
from mcore_bridge_b200.train.presets import hf_config


def test_pattern_language():
    assert _eval_pattern('([0]*3+[1]*1)*2') == [0, 0, 0, 1, 0, 0, 0, 1]
    with pytest.raises(ValueError):
        _eval_pattern('__import__("os")')
    assert tuple_type('(1,2)') == (1, 2)


def test_qwen3_parse():
    kw = hf_to_mcore_config(hf_config('qwen3_tiny'))
    assert kw['num_layers'] == 4 and kw['num_query_groups'] == 2 and kw['kv_channels'] == 64
    assert kw['qk_layernorm'] is True and kw['swiglu'] is True and kw['rotary_base'] == 1000000
    assert kw['untie_embeddings_and_output_weights'] is True and kw['add_qkv_bias'] is False
    cfg = ModelConfig(**kw)
    assert cfg.mcore_model_type == 'gpt' and cfg.gated_linear_unit and not cfg.is_moe_model
    assert cfg.bridge is not None


def test_qwen3_moe_parse():
    kw = hf_to_mcore_config(hf_config('qwen3_moe_tiny'))
    assert 'ffn_hidden_size' not in kw
    assert kw['num_moe_experts'] == 8 and kw['moe_router_topk'] == 2 and kw['moe_ffn_hidden_size'] == 128
    assert kw['moe_router_pre_softmax'] is False
    cfg = ModelConfig(**kw)
    assert cfg.is_moe_model and cfg.moe_layer_pattern() == [1, 1]


def test_deepseek_v3_parse():
    from transformers import DeepseekV3Config
    c = DeepseekV3Config(num_hidden_layers=3, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                         q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                         n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1, moe_intermediate_size=32,
                         intermediate_size=64, first_k_dense_replace=1, n_shared_experts=1, vocab_size=256, scoring_func='sigmoid')
    kw = hf_to_mcore_config(c)
    assert kw['multi_latent_attention'] and kw['moe_router_load_balancing_type'] == 'seq_aux_loss'
    assert kw['moe_layer_freq'] == '[0]*1+[1]*2' and kw['moe_shared_expert_intermediate_size'] == 32
    assert kw['moe_router_score_function'] == 'sigmoid' and kw['moe_router_enable_expert_bias'] is True
    cfg = ModelConfig(**kw)
    assert cfg.moe_layer_pattern() == [0, 1, 1]


def test_deepcopy_shares_bridge():
    import copy
    cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_tiny')))
    c2 = copy.deepcopy(cfg)
    assert c2.bridge is cfg.bridge and c2.num_layers == 4


def test_linear_attention_freq():
    cfg = ModelConfig(**{**hf_to_mcore_config(hf_config('qwen3_tiny')), 'num_layers': 8, 'linear_attention_freq': 4})
    assert cfg.linear_attention_pattern() == [1, 1, 1, 0, 1, 1, 1, 0]


def test_selective_recompute_matches_plain():
    """``recompute_granularity='selective'`` with the mlp / self_attn modules gives the same loss and gradients."""
    import torch
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import init_weights
    ids = torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(0))
    labels = torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(1))
    res = []
    for kw in ({}, dict(recompute_granularity='selective', recompute_modules=['mlp', 'self_attn'])):
        cfg = model_config('qwen3_tiny', params_dtype=torch.float32, **kw)
        m = get_mcore_model(cfg)[0].train()
        init_weights(m, 0.02, 5)
        loss = m(ids, labels=labels).mean()
        loss.backward()
        res.append((loss.detach(), m.decoder.layers[0].mlp.linear_fc1.weight.grad.clone(),
                    m.decoder.layers[1].self_attention.linear_qkv.weight.grad.clone()))
    assert torch.equal(res[0][0], res[1][0])
    assert torch.allclose(res[0][1], res[1][1], atol=1e-7) and torch.allclose(res[0][2], res[1][2], atol=1e-7)
