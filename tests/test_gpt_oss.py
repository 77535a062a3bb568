"""GPT-OSS against ``transformers.GptOssForCausalLM``: learnable softmax sinks, alternating sliding-window layers, YaRN
rope, biased gate and experts (fused, interleaved gate / up storage), clamped quick-GEGLU — logits, gradients of the
biases and a byte-exact checkpoint round trip."""
import torch


def test_gpt_oss_matches_transformers(tmp_path):
    from transformers import AutoConfig, GptOssConfig, GptOssForCausalLM

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    torch.manual_seed(0)
    c = GptOssConfig(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                     intermediate_size=64, num_local_experts=4, num_experts_per_tok=2, vocab_size=256,
                     max_position_embeddings=512, sliding_window=32, tie_word_embeddings=False,
                     layer_types=['sliding_attention', 'full_attention'] * 2)
    hf = GptOssForCausalLM(c).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0 if 'norm' in n else 0.0, 0.05)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    cfg = ModelConfig(**hf_to_mcore_config(AutoConfig.from_pretrained(d)), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], d)
    g = torch.Generator().manual_seed(1)
    ids, labels = torch.randint(0, 256, (2, 96), generator=g), torch.randint(0, 256, (2, 96), generator=g)
    ref = hf(ids).logits
    torch.nn.functional.cross_entropy(ref.view(-1, 256), labels.view(-1)).backward()
    with torch.no_grad():
        assert torch.allclose(model.eval()(ids), ref, atol=2e-5)
    model.train()(ids, labels=labels).mean().backward()
    mlp, hmlp = model.decoder.layers[1].mlp, hf.model.layers[1].mlp

    def close(a, b):
        return ((a - b).norm() / b.norm().clamp_min(1e-12)).item() < 1e-4

    assert close(mlp.router.bias.grad, hmlp.router.bias.grad)
    assert close(mlp.experts.linear_fc2.bias.grad, hmlp.experts.down_proj_bias.grad)
    gb = hmlp.experts.gate_up_proj_bias.grad                         # interleaved (gate, up) pairs
    assert close(mlp.experts.linear_fc1.bias.grad, torch.cat([gb[:, ::2], gb[:, 1::2]], dim=1))
    assert close(model.decoder.layers[0].self_attention.core_attention.softmax_offset.grad,
                 hf.model.layers[0].self_attn.sinks.grad)
    exported, sd = dict(cfg.bridge.export_weights([model])), hf.state_dict()
    assert set(exported) == set(sd)
    for k, v in sd.items():
        assert torch.equal(exported[k], v), k
