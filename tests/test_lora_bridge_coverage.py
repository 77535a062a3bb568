"""Adapter checkpoints beyond the dense / MoE layers: saving under pipeline parallelism (every rank takes part in the
collectives of the save), gated-DeltaNet projections, MTP layers, and the refusal to drop a wrapped module that has no
Hugging Face mapping."""
import json
import os

import pytest
import torch

from dist_utils import run_ranks


def _randomize_lora(model, seed=3):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
            if 'lora_' in n:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)


def _pp_worker(rank, world, out_dir):
    from safetensors.torch import load_file

    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import init_weights
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    ps.initialize_model_parallel(pipeline_model_parallel_size=world)
    cfg = model_config('qwen3_tiny', params_dtype=torch.float32, pipeline_model_parallel_size=world)
    lc = LoraConfig(r=4, lora_alpha=8, target_modules='all-linear')
    models = get_mcore_model(cfg)
    for m in models:
        init_weights(m, 0.05, 1)
    pefts = [get_peft_model(m, lc) for m in models]
    for m in pefts:
        _randomize_lora(m, seed=3 + rank)
    cfg.bridge.save_weights(pefts, out_dir, peft_format=True)        # used to hang: config written by the master only
    saved = load_file(os.path.join(out_dir, 'adapter_model.safetensors'))
    fresh = [get_peft_model(m, lc) for m in get_mcore_model(cfg)]
    cfg.bridge.load_weights(fresh, out_dir, peft_format=True)
    again = dict(cfg.bridge.export_weights(fresh, peft_format=True))
    assert sorted(again) == sorted(saved)
    return all(torch.equal(again[k], saved[k]) for k in saved), sorted(saved)


def test_adapter_save_and_reload_under_pipeline_parallel(tmp_path):
    d = str(tmp_path / 'adapter')
    res = run_ranks(_pp_worker, 2, d)
    assert all(ok for ok, _ in res)
    keys = res[0][1]
    # layers of both stages are in the file
    assert any('.layers.0.' in k for k in keys) and any('.layers.3.' in k for k in keys)
    ac = json.load(open(os.path.join(d, 'adapter_config.json')))
    assert set(ac['target_modules']) == {'q_proj', 'k_proj', 'v_proj', 'o_proj', 'gate_proj', 'up_proj', 'down_proj'}


def _next_config(**kw):
    from transformers import Qwen3NextConfig
    return Qwen3NextConfig(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                           intermediate_size=256, moe_intermediate_size=32, shared_expert_intermediate_size=48,
                           num_experts=8, num_experts_per_tok=2, linear_num_key_heads=2, linear_num_value_heads=4,
                           linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4, vocab_size=256,
                           max_position_embeddings=512, full_attention_interval=4, partial_rotary_factor=0.25,
                           tie_word_embeddings=False, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True, **kw)


def test_gated_delta_net_and_mtp_adapters_round_trip(tmp_path):
    """'all-linear' also wraps the gated-DeltaNet input / output projections and the MTP layer; their factors must be
    exported under the Hugging Face names, reloaded, and give the Hugging Face-style merged model's output."""
    from safetensors.torch import load_file
    from transformers import Qwen3NextForCausalLM

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.train.trainer import init_weights
    from mcore_bridge_b200.tuners import LoraConfig, LoraParallelLinear, get_peft_model
    c = _next_config()
    kw = hf_to_mcore_config(c)
    cfg = ModelConfig(**kw, params_dtype=torch.float32, mtp_num_layers=1)
    model = get_mcore_model(cfg)[0]
    init_weights(model, 0.05, 1)
    d_full, d_ad = str(tmp_path / 'full'), str(tmp_path / 'adapter')
    cfg.bridge.save_weights([model], d_full)
    lc = LoraConfig(r=4, lora_alpha=8, target_modules='all-linear')
    peft = get_peft_model(model, lc)
    wrapped = {n for n, m in peft.named_modules() if isinstance(m, LoraParallelLinear)}
    assert any(n.endswith('self_attention.in_proj') for n in wrapped)
    assert any(n.endswith('self_attention.out_proj') for n in wrapped)
    assert any(n.endswith('eh_proj') for n in wrapped)
    _randomize_lora(peft)
    cfg.bridge.save_weights([peft], d_ad, peft_format=True)
    sd = load_file(os.path.join(d_ad, 'adapter_model.safetensors'))
    lin = 'base_model.model.model.layers.0.linear_attn.'
    for n in ('in_proj_qkvz', 'in_proj_ba', 'out_proj'):
        assert f'{lin}{n}.lora_A.weight' in sd and f'{lin}{n}.lora_B.weight' in sd, n
    assert torch.equal(sd[f'{lin}in_proj_qkvz.lora_A.weight'], sd[f'{lin}in_proj_ba.lora_A.weight'])
    assert 'base_model.model.model.layers.4.eh_proj.lora_B.weight' in sd          # MTP layer follows the decoder
    assert any(k.startswith('base_model.model.model.layers.4.self_attn.q_proj.lora_') for k in sd)
    ac = json.load(open(os.path.join(d_ad, 'adapter_config.json')))
    assert {'in_proj_qkvz', 'in_proj_ba', 'out_proj', 'eh_proj'} <= set(ac['target_modules'])
    # reload into a fresh wrapped model: identical outputs
    model2 = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model2], d_full)
    peft2 = get_peft_model(model2, lc)
    cfg.bridge.load_weights([peft2], d_ad, peft_format=True)
    ids = torch.randint(0, 256, (2, 64), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ours = peft(ids)
        assert torch.allclose(ours, peft2(ids), atol=1e-6)
    # the decoder part applied the Hugging Face way (W + scale * B A) reproduces the logits; the routed experts are
    # stored fused per layer on the Hugging Face side, so their adapters are switched off for this comparison
    with torch.no_grad():
        for n, p in peft.named_parameters():
            if '.experts.' in n and 'lora_B' in n:
                p.zero_()
        ours = peft(ids)
    sd = dict(cfg.bridge.export_weights([peft], peft_format=True))
    hf = Qwen3NextForCausalLM.from_pretrained(d_full).float().eval()
    hsd = hf.state_dict()
    with torch.no_grad():
        for k, a in sd.items():
            if k.endswith('lora_A.weight') and '.layers.4.' not in k and '.experts.' not in k:
                wk = k[len('base_model.model.'):].replace('.lora_A.weight', '.weight')
                hsd[wk].add_(2.0 * sd[k.replace('lora_A', 'lora_B')] @ a)
        assert (hf(ids).logits - ours).abs().max().item() < 1e-4


def test_unmapped_lora_module_is_an_error(tmp_path):
    """A wrapped linear that the slot tables do not know must stop the export instead of being left out."""
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.layers.linear import ReplicatedLinear
    from mcore_bridge_b200.train.presets import hf_config
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_tiny')), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0]
    model.decoder.layers[0].extra_proj = ReplicatedLinear(256, 256, cfg)
    peft = get_peft_model(model, LoraConfig(r=4, lora_alpha=8, target_modules='all-linear'))
    with pytest.raises(NotImplementedError, match='extra_proj'):
        dict(cfg.bridge.export_weights([peft], peft_format=True))
