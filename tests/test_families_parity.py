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


def _sweep_cases():
    common = dict(vocab_size=256, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  max_position_embeddings=512, tie_word_embeddings=False)
    moe = dict(intermediate_size=256, moe_intermediate_size=64, n_routed_experts=4, num_experts_per_tok=2,
               n_shared_experts=1, first_k_dense_replace=1, n_group=1, topk_group=1)
    return common, {
        'llama': ('LlamaConfig', 'LlamaForCausalLM', dict(intermediate_size=256)),
        'qwen2': ('Qwen2Config', 'Qwen2ForCausalLM', dict(intermediate_size=256)),
        'mistral': ('MistralConfig', 'MistralForCausalLM', dict(intermediate_size=256, sliding_window=None)),
        'qwen2_moe': ('Qwen2MoeConfig', 'Qwen2MoeForCausalLM',
                      dict(intermediate_size=256, moe_intermediate_size=64, shared_expert_intermediate_size=96,
                           num_experts=4, num_experts_per_tok=2, decoder_sparse_step=1, mlp_only_layers=[])),
        'ernie4_5': ('Ernie4_5Config', 'Ernie4_5ForCausalLM', dict(intermediate_size=256, head_dim=32)),
        'ernie4_5_moe': ('Ernie4_5_MoeConfig', 'Ernie4_5_MoeForCausalLM',
                         dict(intermediate_size=256, moe_intermediate_size=64, moe_num_experts=4, moe_k=2,
                              moe_num_shared_experts=1, moe_layer_start_index=1, moe_layer_interval=1)),
        'glm4_moe': ('Glm4MoeConfig', 'Glm4MoeForCausalLM', dict(head_dim=32, **moe)),
        'deepseek_v2': ('DeepseekV2Config', 'DeepseekV2ForCausalLM',
                        dict(q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                             **{**moe, 'num_key_value_heads': 4})),
        'dots1': ('Dots1Config', 'Dots1ForCausalLM', dict(head_dim=32, **moe)),       # raw sigmoid scores as weights
        # MLA attention (interleaved rope) + sigmoid-routed MoE with a shared expert
        'glm4_moe_lite': ('Glm4MoeLiteConfig', 'Glm4MoeLiteForCausalLM',
                          dict(q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                               **{**moe, 'num_key_value_heads': 4})),
    }


@pytest.mark.parametrize('name', ['llama', 'qwen2', 'mistral', 'qwen2_moe', 'ernie4_5', 'ernie4_5_moe', 'glm4_moe',
                                  'deepseek_v2', 'dots1', 'glm4_moe_lite'])
def test_generic_family_logits_and_roundtrip(name, tmp_path):
    """The families served by the generic model + bridge pair: logits against Transformers and a byte-exact round trip
    against the checkpoint on disk."""
    import os

    import transformers as tf
    from safetensors.torch import load_file

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    common, cases = _sweep_cases()
    cname, mname, kw = cases[name]
    torch.manual_seed(0)
    hf = getattr(tf, mname)(getattr(tf, cname)(**{**common, **kw})).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0 if 'norm' in n else 0.0, 0.05)
        for n, b in hf.named_buffers():
            if n.endswith('e_score_correction_bias'):
                b.normal_(0, 0.1)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    cfg = ModelConfig(**hf_to_mcore_config(tf.AutoConfig.from_pretrained(d)), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0].eval()
    cfg.bridge.load_weights([model], d)
    ids = torch.randint(0, 256, (2, 64), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        # the MLA path sums in a different order than Transformers: fp32 rounding at the 5th decimal
        assert torch.allclose(model(ids), hf(ids).logits, atol=1e-4 if name == 'glm4_moe_lite' else 3e-5)
    disk = load_file(os.path.join(d, 'model.safetensors'))
    exported = dict(cfg.bridge.export_weights([model]))
    assert set(exported) == set(disk), set(exported) ^ set(disk)
    for k, v in disk.items():
        assert torch.equal(exported[k], v), k


@pytest.mark.parametrize('alias,base', [('kimi_k2', 'deepseek_v3'), ('mimo', 'qwen2'), ('internlm3', 'llama'),
                                        ('deepseek_v3', 'deepseek_v3')])
def test_alias_families_match_their_architecture(alias, base, tmp_path):
    """Model types that reuse another family's architecture (Kimi-K2 = DeepSeek-V3, MiMo = Qwen2 plus MTP layers that
    a plain checkpoint lacks, InternLM3 = Llama): the config parser has to give them the same model, checked by logits
    against the architecture's Transformers class and a byte-exact round trip."""
    import transformers as tf
    common, cases = _sweep_cases()
    cases['deepseek_v3'] = ('DeepseekV3Config', 'DeepseekV3ForCausalLM',
                            dict(q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                                 intermediate_size=256, moe_intermediate_size=64, n_routed_experts=8,
                                 num_experts_per_tok=2, n_shared_experts=1, first_k_dense_replace=1, n_group=2,
                                 topk_group=1, num_key_value_heads=4, routed_scaling_factor=2.5, norm_topk_prob=True))
    cname, mname, kw = cases[base]
    torch.manual_seed(0)
    c = getattr(tf, cname)(**{**common, **kw})
    hf = getattr(tf, mname)(c).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0 if 'norm' in n else 0.0, 0.05)
        for n, b in hf.named_buffers():
            if n.endswith('e_score_correction_bias'):
                b.normal_(0, 0.1)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    c.model_type = alias                                   # what the published config of the alias family says
    kw_mcore = hf_to_mcore_config(c)
    assert kw_mcore.get('hf_model_type', alias) == alias or kw_mcore.get('llm_model_type') == alias
    cfg = ModelConfig(**kw_mcore, params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0].eval()
    cfg.bridge.load_weights([model], d)
    ids = torch.randint(0, 256, (2, 64), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        assert torch.allclose(model(ids), hf(ids).logits, atol=3e-5)
    disk = load_file(os.path.join(d, 'model.safetensors'))
    exported = dict(cfg.bridge.export_weights([model]))
    assert set(exported) == set(disk), set(exported) ^ set(disk)
    for k, v in disk.items():
        assert torch.equal(exported[k], v), k
