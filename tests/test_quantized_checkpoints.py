"""Quantised checkpoints load through the ordinary bridge: MXFP4 experts (GPT-OSS layout) and compressed-tensors
packed int4 experts are dequantised on the fly into the same parameters a bf16 checkpoint would give."""
import json
import os

import torch
from safetensors.torch import load_file, save_file


def test_mxfp4_quantise_dequantise_is_consistent():
    from mcore_bridge_b200.utils.dequantizer import MxFp4Dequantizer, quantize_mxfp4
    torch.manual_seed(0)
    w = torch.randn(3, 8, 64) * 0.3
    blocks, scales = quantize_mxfp4(w)
    assert blocks.shape == (3, 8, 2, 16) and scales.shape == (3, 8, 2)
    deq = MxFp4Dequantizer().convert(blocks, scales, torch.float32)
    assert deq.shape == w.shape
    # e2m1 has a relative step of at most 1/3 around a value; values are representable after one round trip
    assert (deq - w).abs().max() <= 0.26 * w.abs().reshape(3, 8, 2, 32).amax(-1).max()
    b2, s2 = quantize_mxfp4(deq)
    assert torch.equal(MxFp4Dequantizer().convert(b2, s2, torch.float32), deq)


def test_gpt_oss_mxfp4_checkpoint_loads(tmp_path):
    from transformers import AutoConfig, GptOssConfig, GptOssForCausalLM

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.utils.dequantizer import MxFp4Dequantizer, quantize_mxfp4
    torch.manual_seed(0)
    c = GptOssConfig(num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                     intermediate_size=64, num_local_experts=4, num_experts_per_tok=2, vocab_size=256,
                     max_position_embeddings=512, sliding_window=32, tie_word_embeddings=False,
                     layer_types=['sliding_attention', 'full_attention'])
    hf = GptOssForCausalLM(c).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0 if 'norm' in n else 0.0, 0.05)
    d_ref, d_q = str(tmp_path / 'bf16'), str(tmp_path / 'mxfp4')
    hf.save_pretrained(d_ref)
    sd = load_file(os.path.join(d_ref, 'model.safetensors'))
    # store the experts the way the published MXFP4 checkpoints do: output-major, 32-value blocks along the input dim
    qsd, deq = {}, MxFp4Dequantizer()
    for k, v in sd.items():
        if k.endswith('experts.gate_up_proj') or k.endswith('experts.down_proj'):
            blocks, scales = quantize_mxfp4(v.transpose(1, 2).contiguous())
            qsd[k + '_blocks'], qsd[k + '_scales'] = blocks, scales
            sd[k] = deq.convert(blocks, scales, torch.float32).transpose(1, 2).contiguous()   # what loading must give
        else:
            qsd[k] = v
    os.makedirs(d_q)
    save_file(qsd, os.path.join(d_q, 'model.safetensors'))
    save_file(sd, os.path.join(d_ref, 'model.safetensors'))
    cfg = ModelConfig(**hf_to_mcore_config(AutoConfig.from_pretrained(d_ref)), params_dtype=torch.float32)
    m_ref, m_q = get_mcore_model(cfg)[0], get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([m_ref], d_ref)
    cfg.bridge.load_weights([m_q], d_q)
    for (n, a), (_, b) in zip(m_ref.named_parameters(), m_q.named_parameters()):
        assert torch.equal(a, b), n
    ids = torch.randint(0, 256, (2, 48), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        assert torch.equal(m_ref.eval()(ids), m_q.eval()(ids))


def test_compressed_tensors_int4_experts_load(tmp_path):
    from transformers import Qwen3MoeForCausalLM

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.train.presets import hf_config
    from mcore_bridge_b200.utils.dequantizer import pack_int_weights
    torch.manual_seed(0)
    c = hf_config('qwen3_moe_tiny')
    hf = Qwen3MoeForCausalLM(c).float()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0, 0.05)
    d_ref, d_q = str(tmp_path / 'plain'), str(tmp_path / 'int4')
    hf.save_pretrained(d_ref)
    files = [f for f in os.listdir(d_ref) if f.endswith('.safetensors')]
    assert files == ['model.safetensors']
    sd = load_file(os.path.join(d_ref, 'model.safetensors'))
    group, bits = 32, 4
    qsd, n_packed = {}, 0
    for k, v in list(sd.items()):
        if '.experts.' in k and k.endswith('_proj.weight'):
            rows, cols = v.shape
            g = v.reshape(rows, cols // group, group)
            scale = (g.abs().amax(-1) / 7.0).clamp(min=1e-8)
            q = torch.clamp(torch.round(g / scale.unsqueeze(-1)), -8, 7).to(torch.int64).reshape(rows, cols)
            mod = k[:-len('.weight')]
            qsd[mod + '.weight_packed'] = pack_int_weights(q, bits)
            qsd[mod + '.weight_scale'] = scale
            qsd[mod + '.weight_shape'] = torch.tensor([rows, cols], dtype=torch.int64)
            sd[k] = (q.reshape(rows, cols // group, group).float() * scale.unsqueeze(-1)).reshape(rows, cols)
            n_packed += 1
        else:
            qsd[k] = v
    assert n_packed > 0
    os.makedirs(d_q)
    save_file(qsd, os.path.join(d_q, 'model.safetensors'))
    save_file(sd, os.path.join(d_ref, 'model.safetensors'))
    cfg_json = json.load(open(os.path.join(d_ref, 'config.json')))
    cfg_json['quantization_config'] = {'quant_method': 'compressed-tensors', 'config_groups': {
        'group_0': {'weights': {'num_bits': bits, 'group_size': group, 'symmetric': True, 'type': 'int'}}}}
    json.dump(cfg_json, open(os.path.join(d_q, 'config.json'), 'w'))
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    m_ref, m_q = get_mcore_model(cfg)[0], get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([m_ref], d_ref)
    cfg.bridge.load_weights([m_q], d_q)
    for (n, a), (_, b) in zip(m_ref.named_parameters(), m_q.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6, rtol=0), n
