"""LoRA: injection, adapter math vs merged weights, PEFT-format round-trip, TP=2 export equality."""
import json
import os

import torch

from dist_utils import run_ranks


def _build(tp=1, sp=False, name='qwen3_tiny', seed=0):
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.train.presets import hf_config
    from mcore_bridge_b200.train.trainer import init_weights
    cfg = ModelConfig(**hf_to_mcore_config(hf_config(name)), params_dtype=torch.float32,
                      tensor_model_parallel_size=tp, sequence_parallel=sp)
    model = get_mcore_model(cfg)[0]
    init_weights(model, 0.05, seed + 1)
    return cfg, model


def _randomize_lora(model, seed=3):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if 'lora_' in n:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)


def test_inject_forward_merge(tmp_path):
    from mcore_bridge_b200.tuners import LoraConfig, LoraParallelLinear, get_peft_model
    cfg, model = _build()
    ids = torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        base_out = model(ids)
    peft = get_peft_model(model, LoraConfig(r=8, lora_alpha=16, target_modules=['linear_qkv', 'linear_proj', 'linear_fc1',
                                                                               'linear_fc2']))
    n_lora = sum(isinstance(m, LoraParallelLinear) for m in peft.modules())
    assert n_lora == 4 * 4
    assert all(('lora_' in n) == p.requires_grad for n, p in peft.named_parameters())
    with torch.no_grad():
        assert torch.allclose(peft(ids), base_out, atol=1e-6)   # B = 0 at init
    _randomize_lora(peft)
    with torch.no_grad():
        out = peft(ids)
        assert (out - base_out).abs().max() > 1e-4
        peft.merge_adapter()
        merged = peft(ids)
        assert torch.allclose(out, merged, atol=2e-5)
        peft.unmerge_adapter()
        assert torch.allclose(peft(ids), out, atol=2e-5)
    loss = peft(ids, labels=ids).mean()
    loss.backward()
    for n, p in peft.named_parameters():
        if 'lora_' in n:
            assert p.grad is not None and torch.isfinite(p.grad).all(), n


def test_peft_format_roundtrip(tmp_path):
    from safetensors.torch import load_file

    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    cfg, model = _build(name='qwen3_moe_tiny')
    lc = LoraConfig(r=8, lora_alpha=32, target_modules='all-linear')
    peft = get_peft_model(model, lc)
    _randomize_lora(peft)
    # fused projections share lora_A in HF format: nothing to enforce on export (A is exported once per HF name)
    d = str(tmp_path / 'adapter')
    cfg.bridge.save_weights([peft], d, peft_format=True)
    sd = load_file(os.path.join(d, 'adapter_model.safetensors'))
    ac = json.load(open(os.path.join(d, 'adapter_config.json')))
    assert ac['r'] == 8 and ac['lora_alpha'] == 32 and ac['peft_type'] == 'LORA'
    assert set(ac['target_modules']) >= {'q_proj', 'k_proj', 'v_proj', 'o_proj', 'gate_proj', 'up_proj', 'down_proj'}
    k = 'base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight'
    assert k in sd and sd[k].shape == (4 * 64, 8)
    assert 'base_model.model.model.layers.1.mlp.experts.3.down_proj.lora_A.weight' in sd
    # load into a fresh model and compare outputs
    cfg2, model2 = _build(name='qwen3_moe_tiny')
    peft2 = get_peft_model(model2, lc)
    cfg2.bridge.load_weights([peft2], d, peft_format=True)
    ids = torch.randint(0, 1024, (2, 32), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        assert torch.allclose(peft(ids), peft2(ids), atol=1e-6)


def test_hf_peft_semantics(tmp_path):
    """The exported adapter applied the Hugging Face way (W + scale * B A on q/k/v/o/gate/up/down) gives our output."""
    from transformers import Qwen3ForCausalLM

    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    from mcore_bridge_b200.train.presets import hf_config
    cfg, model = _build()
    d_full = str(tmp_path / 'full')
    cfg.bridge.save_weights([model], d_full)
    peft = get_peft_model(model, LoraConfig(r=4, lora_alpha=8, target_modules='all-linear'))
    _randomize_lora(peft)
    sd = dict(cfg.bridge.export_weights([peft], peft_format=True))
    hf = Qwen3ForCausalLM.from_pretrained(d_full).float().eval()
    hsd = hf.state_dict()
    scale = 8 / 4
    with torch.no_grad():
        for k, a in sd.items():
            if k.endswith('lora_A.weight'):
                b = sd[k.replace('lora_A', 'lora_B')]
                wk = k[len('base_model.model.'):].replace('.lora_A.weight', '.weight')
                hsd[wk].add_(scale * b @ a)
    ids = torch.randint(0, 1024, (2, 48), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        assert torch.allclose(hf(ids).logits, peft(ids), atol=2e-5)


def _tp_worker(rank, world, sp):
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.parallel.random import model_parallel_manual_seed
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    ps.initialize_model_parallel(tensor_model_parallel_size=2)
    model_parallel_manual_seed(7)
    cfg, model = _build(tp=2, sp=sp)
    peft = get_peft_model(model, LoraConfig(r=4, lora_alpha=8, target_modules='all-linear'))
    ids = torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        for n, p in peft.named_parameters():
            if 'lora_B' in n:
                p.normal_(0, 0.05)
    sd = dict(cfg.bridge.export_weights([peft], peft_format=True))
    full = dict(cfg.bridge.export_weights([peft]))
    with torch.no_grad():
        out = peft(ids, runtime_gather_output=True)
    return {k: v.clone() for k, v in sd.items()}, {k: v.clone() for k, v in full.items()}, out


def test_tp2_adapter_export_matches_dense_application():
    for sp in (False, True):
        res = run_ranks(_tp_worker, 2, sp)
        sd0, full0, out0 = res[0]
        sd1, full1, out1 = res[1]
        assert sorted(sd0) == sorted(sd1) and all(torch.equal(sd0[k], sd1[k]) for k in sd0)
        assert torch.allclose(out0, out1, atol=1e-6)
        # apply the exported adapter to the exported full weights and run the single-process model
        from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
        from mcore_bridge_b200.train.presets import hf_config
        merged = {k: v.clone() for k, v in full0.items()}
        for k, a in sd0.items():
            if k.endswith('lora_A.weight'):
                b = sd0[k.replace('lora_A', 'lora_B')]
                merged[k[len('base_model.model.'):].replace('.lora_A.weight', '.weight')] += 2.0 * b @ a
        cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_tiny')), params_dtype=torch.float32)
        model = get_mcore_model(cfg)[0]
        from mcore_bridge_b200.utils.safetensors import LazyTensor
        for _ in cfg.bridge._convert([model], {k: LazyTensor(tensor=v) for k, v in merged.items()}, True):
            pass
        ids = torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(0))
        with torch.no_grad():
            assert torch.allclose(model(ids), out0, atol=3e-5)
