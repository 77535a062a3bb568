"""Tiny Qwen3 / Qwen3-MoE: HF safetensors -> model -> HF safetensors byte-equal, logits and one AdamW step vs Transformers."""
import os

import pytest
import torch
from safetensors.torch import load_file

from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
from mcore_bridge_b200.train.presets import hf_config


def _hf_model(name, std=0.02):
    from transformers import Qwen3ForCausalLM, Qwen3MoeForCausalLM
    torch.manual_seed(0)
    c = hf_config(name)
    cls = Qwen3MoeForCausalLM if 'moe' in name else Qwen3ForCausalLM
    m = cls(c).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.normal_(0, std)
            else:
                p.normal_(1.0, 0.1)   # norm weights away from 1 so that a swapped norm shows up
    return c, m


@pytest.mark.parametrize('name', ['qwen3_tiny', 'qwen3_moe_tiny'])
def test_roundtrip_and_logits(name, tmp_path):
    c, hf = _hf_model(name)
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    hf.save_pretrained(d1)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], d1)
    ids = torch.randint(0, 1024, (2, 128), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ref = hf(ids).logits
        out = model(ids)
    assert (ref - out).abs().max().item() < 1e-5
    cfg.bridge.save_weights([model], d2)
    a, b = load_file(os.path.join(d1, 'model.safetensors')), load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(a) == sorted(b)
    for k in a:
        assert torch.equal(a[k], b[k]), k
    assert os.path.exists(os.path.join(d2, 'config.json'))


def test_loss_and_adamw_step_match_hf(tmp_path):
    c, hf = _hf_model('qwen3_tiny')
    d1 = str(tmp_path / 'a')
    hf.save_pretrained(d1)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], d1)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1024, (2, 128), generator=g)
    labels = torch.randint(0, 1024, (2, 128), generator=g)
    hf.train()
    opt_h = torch.optim.AdamW(hf.parameters(), lr=1e-3, weight_decay=0.0)
    opt_m = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.0)
    logits = hf(ids).logits
    loss_h = torch.nn.functional.cross_entropy(logits.view(-1, 1024), labels.view(-1))
    loss_h.backward()
    opt_h.step()
    loss_m = model(ids, labels=labels).mean()
    loss_m.backward()
    opt_m.step()
    assert abs(loss_h.item() - loss_m.item()) < 1e-5
    exported = dict(cfg.bridge.export_weights([model]))
    hf_sd = hf.state_dict()
    # the first Adam update is lr * g / (|g| + eps): where g is ~0 its sign is rounding noise, so a handful of
    # elements may differ by up to 2 * lr; everything else must agree closely
    for k, v in exported.items():
        diff = (v - hf_sd[k]).abs()
        assert diff.max().item() <= 2.1e-3, k
        assert (diff > 2e-5).float().mean().item() < 2e-3, k


def test_sharded_save_index(tmp_path):
    c, hf = _hf_model('qwen3_tiny')
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    hf.save_pretrained(d1)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], d1)
    cfg.bridge.save_weights([model], d2, max_shard_size='2MB')
    import json
    idx = json.load(open(os.path.join(d2, 'model.safetensors.index.json')))
    files = set(idx['weight_map'].values())
    assert len(files) > 1 and all(os.path.exists(os.path.join(d2, f)) for f in files)
    from transformers import Qwen3ForCausalLM
    re = Qwen3ForCausalLM.from_pretrained(d2).float()
    for k, v in hf.state_dict().items():
        assert torch.equal(v, re.state_dict()[k]), k
    # converter hook renames on the way out
    names = [k for k, _ in cfg.bridge.export_weights([model], converter=lambda k, v: ('x.' + k, v))]
    assert all(n.startswith('x.') for n in names)
