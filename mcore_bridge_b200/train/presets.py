"""Named model shapes used by the benchmarks and tests, expressed as Hugging Face configs so they go through
the same ``hf_to_mcore_config`` -> ``ModelConfig`` path a user takes."""
from __future__ import annotations

from typing import Any, Dict


def hf_config(name: str, **overrides):
    from transformers import Qwen3Config, Qwen3MoeConfig
    if name == 'qwen3_tiny':
        kw = dict(num_hidden_layers=4, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                  intermediate_size=768, vocab_size=1024, rope_theta=1e6, rms_norm_eps=1e-6,
                  tie_word_embeddings=False, max_position_embeddings=4096)
        kw.update(overrides)
        return Qwen3Config(**kw)
    if name == 'qwen3_8b':
        kw = dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                  intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                  tie_word_embeddings=False, max_position_embeddings=40960)
        kw.update(overrides)
        return Qwen3Config(**kw)
    if name == 'qwen3_moe_tiny':
        kw = dict(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                  intermediate_size=768, moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                  vocab_size=1024, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                  max_position_embeddings=4096, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])
        kw.update(overrides)
        return Qwen3MoeConfig(**kw)
    if name == 'qwen3_30b_a3b':
        kw = dict(num_hidden_layers=48, hidden_size=2048, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                  intermediate_size=6144, moe_intermediate_size=768, num_experts=128, num_experts_per_tok=8,
                  vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                  max_position_embeddings=40960, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
                  router_aux_loss_coef=1e-3)
        kw.update(overrides)
        return Qwen3MoeConfig(**kw)
    raise ValueError(f'unknown preset {name}')


def model_config(name: str, hf_overrides: Dict[str, Any] = None, **config_overrides):
    from ..config import ModelConfig, hf_to_mcore_config
    kw = hf_to_mcore_config(hf_config(name, **(hf_overrides or {})))
    kw.update(config_overrides)
    return ModelConfig(**kw)
