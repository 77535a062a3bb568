"""DeepSeek-V3 (MLA, sigmoid group-limited routing, shared expert) and GLM-5 style DSA sparse attention against
the Transformers implementations; bridge round-trip for both."""
import os

import torch
from safetensors.torch import load_file

from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config


def _init(hf):
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.06) if p.dim() >= 2 else p.normal_(1.0, 0.1)
        for n, b in hf.named_buffers():
            if 'e_score_correction_bias' in n:
                b.normal_(0, 0.1)


def _roundtrip(hf, c, tmp_path, ids, atol):
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    hf.save_pretrained(d1)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0].eval()
    cfg.bridge.load_weights([model], d1)
    with torch.no_grad():
        ref, out = hf(ids).logits, model(ids)
    assert (ref - out).abs().max().item() < atol
    cfg.bridge.save_weights([model], d2)
    a, b = load_file(os.path.join(d1, 'model.safetensors')), load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(a) == sorted(b) and all(torch.equal(a[k], b[k]) for k in a)
    return cfg, model


def test_deepseek_v3(tmp_path):
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    torch.manual_seed(0)
    c = DeepseekV3Config(num_hidden_layers=3, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                         q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                         n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1, moe_intermediate_size=32,
                         intermediate_size=64, first_k_dense_replace=1, n_shared_experts=1, vocab_size=256,
                         scoring_func='sigmoid', routed_scaling_factor=2.5, norm_topk_prob=True,
                         max_position_embeddings=512, rope_interleave=True, tie_word_embeddings=False)
    hf = DeepseekV3ForCausalLM(c).float().eval()
    _init(hf)
    ids = torch.randint(0, 256, (2, 48), generator=torch.Generator().manual_seed(0))
    cfg, model = _roundtrip(hf, c, tmp_path, ids, 2e-5)
    assert cfg.multi_latent_attention and cfg.moe_layer_pattern() == [0, 1, 1]


def test_glm_moe_dsa_sparse_attention(tmp_path):
    from transformers import GlmMoeDsaConfig, GlmMoeDsaForCausalLM
    torch.manual_seed(0)
    c = GlmMoeDsaConfig(num_hidden_layers=3, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                        q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                        n_routed_experts=8, num_experts_per_tok=2, n_group=1, topk_group=1, moe_intermediate_size=32,
                        intermediate_size=64, mlp_layer_types=['dense', 'sparse', 'sparse'], n_shared_experts=1,
                        vocab_size=256, routed_scaling_factor=2.5, norm_topk_prob=True, max_position_embeddings=512,
                        tie_word_embeddings=False, index_n_heads=4, index_head_dim=16, index_topk=8)
    c._attn_implementation = 'eager'   # the sdpa path of the HF model drops the causal mask from the indexer
    hf = GlmMoeDsaForCausalLM(c).float().eval()
    _init(hf)
    ids = torch.randint(0, 256, (1, 40), generator=torch.Generator().manual_seed(0))
    cfg, model = _roundtrip(hf, c, tmp_path, ids, 2e-4)
    assert cfg.experimental_attention_variant == 'dsa' and cfg.dsa_indexer_topk == 8


def test_dsa_indexer_loss_trains_indexer():
    from mcore_bridge_b200.train.trainer import init_weights
    from transformers import GlmMoeDsaConfig
    c = GlmMoeDsaConfig(num_hidden_layers=1, hidden_size=64, num_attention_heads=2, num_key_value_heads=2,
                        q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                        n_routed_experts=4, num_experts_per_tok=2, n_group=1, topk_group=1, moe_intermediate_size=16,
                        intermediate_size=32, mlp_layer_types=['dense'], n_shared_experts=1, vocab_size=64,
                        max_position_embeddings=128, index_n_heads=2, index_head_dim=16, index_topk=4)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32, dsa_indexer_loss_coeff=0.1)
    model = get_mcore_model(cfg)[0].train()
    init_weights(model, 0.1, 3)
    ids = torch.randint(0, 64, (1, 32))
    model(ids, labels=ids).mean().backward()
    idx = model.decoder.layers[0].self_attention.indexer
    assert idx.linear_wk.weight.grad is not None and idx.linear_wk.weight.grad.abs().sum() > 0
    assert model.decoder.layers[0].self_attention.indexer_loss is not None


def test_dsa_gather_path_equals_dense_path(monkeypatch):
    """The weight-absorbed, gather-based sparse attention (the long-sequence path) gives the same logits and
    gradients as the dense-masked formulation, on a packed batch."""
    from transformers import GlmMoeDsaConfig

    from mcore_bridge_b200.layers.context import PackedSeqParams
    from mcore_bridge_b200.train.trainer import init_weights
    c = GlmMoeDsaConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=4,
                        q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                        n_routed_experts=4, num_experts_per_tok=2, n_group=1, topk_group=1, moe_intermediate_size=16,
                        intermediate_size=32, mlp_layer_types=['dense', 'dense'], n_shared_experts=1, vocab_size=64,
                        max_position_embeddings=128, index_n_heads=2, index_head_dim=16, index_topk=6)
    ids = torch.randint(0, 64, (1, 48), generator=torch.Generator().manual_seed(2))
    cu = torch.tensor([0, 20, 48], dtype=torch.int32)
    pos = torch.cat([torch.arange(20), torch.arange(28)]).reshape(1, -1)
    psp = PackedSeqParams(cu_seqlens_q=cu, cu_seqlens_kv=cu, max_seqlen_q=28, max_seqlen_kv=28)
    res = []
    for min_t in ('100000', '0'):
        monkeypatch.setenv('MCB200_DSA_GATHER_MIN_T', min_t)
        cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
        model = get_mcore_model(cfg)[0].train()
        init_weights(model, 0.1, 3)
        attn = model.decoder.layers[0].self_attention
        assert attn._use_gather_path(48) == (min_t == '0')
        loss = model(ids, position_ids=pos, labels=ids, packed_seq_params=psp).mean()
        loss.backward()
        res.append((loss.detach(), attn.linear_kv_up_proj.weight.grad.clone(),
                    attn.linear_kv_down_proj.weight.grad.clone(), attn.linear_q_up_proj.weight.grad.clone(),
                    attn.linear_kv_up_proj.layer_norm_weight.grad.clone()))
    assert abs(res[0][0].item() - res[1][0].item()) < 1e-5
    for a, b in zip(res[0][1:], res[1][1:]):
        assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()


def test_dsa_gather_path_with_lora_equals_dense_path(monkeypatch):
    """With LoRA adapters on every linear the weight-absorbed path uses base weight + the adapter's low-rank update of
    the key / value up projection, and the indexer still receives the normalised query latent: same loss and same
    adapter gradients as the dense-masked formulation."""
    from transformers import GlmMoeDsaConfig

    from mcore_bridge_b200.layers.context import PackedSeqParams
    from mcore_bridge_b200.train.trainer import init_weights
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    c = GlmMoeDsaConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=4,
                        q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                        n_routed_experts=4, num_experts_per_tok=2, n_group=1, topk_group=1, moe_intermediate_size=16,
                        intermediate_size=32, mlp_layer_types=['dense', 'dense'], n_shared_experts=1, vocab_size=64,
                        max_position_embeddings=128, index_n_heads=2, index_head_dim=16, index_topk=6)
    ids = torch.randint(0, 64, (1, 48), generator=torch.Generator().manual_seed(2))
    cu = torch.tensor([0, 20, 48], dtype=torch.int32)
    pos = torch.cat([torch.arange(20), torch.arange(28)]).reshape(1, -1)
    psp = PackedSeqParams(cu_seqlens_q=cu, cu_seqlens_kv=cu, max_seqlen_q=28, max_seqlen_kv=28)
    res = []
    for min_t in ('100000', '0'):
        monkeypatch.setenv('MCB200_DSA_GATHER_MIN_T', min_t)
        cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
        model = get_mcore_model(cfg)[0]
        init_weights(model, 0.1, 3)
        peft = get_peft_model(model, LoraConfig(r=4, lora_alpha=8, target_modules='all-linear')).train()
        g = torch.Generator().manual_seed(9)
        with torch.no_grad():
            for n, p in sorted(peft.named_parameters(), key=lambda kv: kv[0]):
                if 'lora_' in n:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.1)
        loss = peft(ids, position_ids=pos, labels=ids, packed_seq_params=psp).mean()
        loss.backward()
        # the indexer is not trained through this loss: its adapters get no gradient
        grads = {n: p.grad.clone() for n, p in peft.named_parameters()
                 if 'lora_' in n and 'layers.0.self_attention' in n and p.grad is not None}
        assert any('linear_kv_up_proj.lora_B' in n for n in grads) and all(g_.abs().sum() > 0 for g_ in grads.values())
        res.append((loss.detach(), grads))
    assert abs(res[0][0].item() - res[1][0].item()) < 1e-5
    for n, g_ in res[0][1].items():
        assert torch.allclose(g_, res[1][1][n], atol=2e-5), (n, (g_ - res[1][1][n]).abs().max())
