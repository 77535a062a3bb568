"""Text families with their own modules or key layouts (GLM-4, OLMoE, MiniMax-M2): logits equal Transformers and the
safetensors round trip is byte-equal."""
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


def _glm4():
    from transformers import Glm4Config, Glm4ForCausalLM
    c = Glm4Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=32, partial_rotary_factor=0.5,
                   max_position_embeddings=256, pad_token_id=0, tie_word_embeddings=False, attention_bias=True)
    return c, Glm4ForCausalLM(c)


def _olmoe():
    from transformers import OlmoeConfig, OlmoeForCausalLM
    c = OlmoeConfig(vocab_size=512, hidden_size=128, intermediate_size=64, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=4, num_experts=8, num_experts_per_tok=2,
                    max_position_embeddings=256, pad_token_id=0, norm_topk_prob=False)
    return c, OlmoeForCausalLM(c)


def _minimax_m2():
    from transformers import MiniMaxM2Config, MiniMaxM2ForCausalLM
    c = MiniMaxM2Config(vocab_size=512, hidden_size=128, intermediate_size=64, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_local_experts=8,
                        num_experts_per_tok=2, max_position_embeddings=256, rotary_dim=16, use_qk_norm=True,
                        pad_token_id=0)
    return c, MiniMaxM2ForCausalLM(c)


@pytest.mark.parametrize('build', [_glm4, _olmoe, _minimax_m2])
def test_family_logits_and_roundtrip(build, tmp_path):
    torch.manual_seed(0)
    c, hf = build()
    hf = _randomise(hf.float().eval())
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    hf.save_pretrained(d1)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0].eval()
    cfg.bridge.load_weights([model], d1)
    ids = torch.randint(0, 512, (2, 64), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ref = hf(ids).logits
        out = model(ids)
    assert (ref - out).abs().max().item() < 2e-5
    cfg.bridge.save_weights([model], d2)
    a, b = load_file(os.path.join(d1, 'model.safetensors')), load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(a) == sorted(b)
    for k in a:
        assert torch.equal(a[k], b[k]), k
