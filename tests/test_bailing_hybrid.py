"""Ling / Ring hybrid (lightning attention + MLA): layer pattern from the HF config, the lightning layer equals the
token-by-token recurrence, and the checkpoint round trip is lossless."""
import os

import torch
from safetensors.torch import load_file

from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config


def _hf_config():
    from transformers import PretrainedConfig
    c = PretrainedConfig()
    c.model_type = 'bailing_hybrid'
    c.architectures = ['BailingMoeV2_5ForCausalLM']
    for k, v in dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=5,
                     num_attention_heads=4, num_key_value_heads=4, head_dim=16, max_position_embeddings=256,
                     rms_norm_eps=1e-6, rope_theta=10000.0, layer_group_size=2, group_norm_size=2,
                     q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                     num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, num_shared_experts=1,
                     first_k_dense_replace=1, n_group=1, topk_group=1, routed_scaling_factor=1.0,
                     norm_topk_prob=True, tie_word_embeddings=False, use_qk_norm=True, hidden_act='silu',
                     partial_rotary_factor=0.5).items():
        setattr(c, k, v)
    return c


def test_pattern_forward_and_roundtrip(tmp_path):
    torch.manual_seed(0)
    c = _hf_config()
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    assert cfg.linear_attention_pattern() == [1, 0, 1, 0, 0]          # groups of 2, tail layer is full attention
    model = get_mcore_model(cfg)[0]
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0, 0.1)
    names = dict(model.named_modules())
    from mcore_bridge_b200.layers.lightning_attention import LightningAttention
    from mcore_bridge_b200.layers.mla import MLASelfAttention
    assert isinstance(names['decoder.layers.0.self_attention'], LightningAttention)
    assert isinstance(names['decoder.layers.1.self_attention'], MLASelfAttention)
    ids = torch.randint(0, 256, (2, 32), generator=torch.Generator().manual_seed(1))
    out = model(ids)
    assert torch.isfinite(out).all()
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    cfg.bridge.save_weights([model], d1)
    sd = load_file(os.path.join(d1, 'model.safetensors'))
    assert 'model.layers.0.attention.query_key_value.weight' in sd and 'model.layers.0.attention.g_norm.weight' in sd
    assert 'model.word_embeddings.weight' in sd
    model2 = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model2], d1)
    with torch.no_grad():
        out2 = model2(ids)
    assert torch.equal(out.detach(), out2)
    cfg.bridge.save_weights([model2], d2)
    sd2 = load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(sd) == sorted(sd2) and all(torch.equal(sd[k], sd2[k]) for k in sd)


def test_lightning_layer_matches_recurrence():
    from mcore_bridge_b200.ops import gdn as G
    torch.manual_seed(2)
    T, h, d = 40, 3, 8
    q, k, v = (torch.randn(T, h, d) for _ in range(3))
    decay = -torch.rand(h) * 0.3
    cu = torch.tensor([0, 15, 40], dtype=torch.int32)
    o = G.simple_gla(q, k, v, decay, cu)
    ref = torch.zeros_like(o)
    for s, e in ((0, 15), (15, 40)):
        S = torch.zeros(h, d, d)
        for t in range(s, e):
            S = S * decay.exp()[:, None, None] + k[t][:, :, None] * v[t][:, None, :]
            ref[t] = torch.einsum('hkv,hk->hv', S, q[t] * d ** -0.5)
    assert (o - ref).abs().max().item() < 1e-4
