"""Qwen3-Next hybrid (gated DeltaNet + gated attention + MoE with gated shared expert) vs Transformers; gated-delta-rule
chunked form vs the token-by-token recurrence, packed sequences included."""
import os

import torch
from safetensors.torch import load_file

from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
from mcore_bridge_b200.ops import gdn


def test_chunk_equals_recurrent_with_packing():
    torch.manual_seed(0)
    T, h, dk, dv = 200, 3, 16, 24
    q = gdn.l2norm(torch.randn(T, h, dk))
    k = gdn.l2norm(torch.randn(T, h, dk))
    v = torch.randn(T, h, dv)
    g = -torch.rand(T, h) * 0.5
    beta = torch.rand(T, h)
    cu = torch.tensor([0, 70, 71, 200], dtype=torch.int32)
    for c in (None, cu):
        a = gdn.recurrent_gated_delta_rule(q, k, v, g, beta, c)
        b = gdn.chunk_gated_delta_rule(q, k, v, g, beta, c, chunk=64)
        assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()
    # a boundary resets the state: the packed result equals running each piece alone
    whole = gdn.chunk_gated_delta_rule(q, k, v, g, beta, cu)
    piece = gdn.chunk_gated_delta_rule(q[71:], k[71:], v[71:], g[71:], beta[71:], None)
    assert torch.allclose(whole[71:], piece, atol=1e-6)


def test_chunk_rule_matches_transformers_reference():
    from transformers.models.qwen3_next.modeling_qwen3_next import torch_chunk_gated_delta_rule
    torch.manual_seed(1)
    B, T, h, dk, dv = 1, 130, 2, 16, 16
    q, k, v = torch.randn(B, T, h, dk), torch.randn(B, T, h, dk), torch.randn(B, T, h, dv)
    g, beta = -torch.rand(B, T, h), torch.rand(B, T, h)
    ref, _ = torch_chunk_gated_delta_rule(q, k, v, g=g, beta=beta, use_qk_l2norm_in_kernel=True)
    ours = gdn.chunk_gated_delta_rule(gdn.l2norm(q[0]), gdn.l2norm(k[0]), v[0], g[0], beta[0])
    assert torch.allclose(ref[0], ours, atol=2e-5)


def test_causal_conv_packed():
    torch.manual_seed(2)
    x, w = torch.randn(50, 6), torch.randn(6, 4)
    cu = torch.tensor([0, 20, 50], dtype=torch.int32)
    y = gdn.causal_conv1d_silu(x, w, None, cu)
    assert torch.allclose(y[20:], gdn.causal_conv1d_silu(x[20:], w), atol=1e-6)
    ref = sum(w[:, j] * torch.nn.functional.pad(x[:20], (0, 0, 3, 0))[j:j + 20] for j in range(4))
    assert torch.allclose(y[:20], torch.nn.functional.silu(ref), atol=1e-5)


def test_qwen3_next_hf_parity(tmp_path):
    from transformers import Qwen3NextConfig, Qwen3NextForCausalLM
    torch.manual_seed(0)
    c = Qwen3NextConfig(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                        intermediate_size=256, moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=8,
                        num_experts_per_tok=2, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                        linear_value_head_dim=16, linear_conv_kernel_dim=4, vocab_size=256, max_position_embeddings=512,
                        full_attention_interval=4, partial_rotary_factor=0.25, tie_word_embeddings=False,
                        decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
    hf = Qwen3NextForCausalLM(c).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if 'A_log' in n or 'dt_bias' in n:
                continue
            p.normal_(0, 0.08) if p.dim() >= 2 else p.normal_(0.0, 0.1)
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    hf.save_pretrained(d1)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    assert cfg.linear_attention_pattern() == [1, 1, 1, 0] and cfg.attention_output_gate
    model = get_mcore_model(cfg)[0].eval()
    cfg.bridge.load_weights([model], d1)
    ids = torch.randint(0, 256, (2, 100), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        assert (hf(ids).logits - model(ids)).abs().max().item() < 5e-5
    cfg.bridge.save_weights([model], d2)
    a, b = load_file(os.path.join(d1, 'model.safetensors')), load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(a) == sorted(b) and all(torch.equal(a[k], b[k]) for k in a)
