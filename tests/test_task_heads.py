"""Task heads of the generic model: sequence classification (score head round-trips through the bridge and matches
Transformers), embedding (L2-normalised hidden states) and the generative reranker (yes/no logit difference)."""
import os

import torch
from safetensors.torch import load_file

from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
from mcore_bridge_b200.train.presets import hf_config


def _hf_base(cls):
    torch.manual_seed(0)
    c = hf_config('qwen3_tiny')
    c.num_labels = 3
    c.pad_token_id = 0
    m = cls(c).float().eval()
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.02) if p.dim() >= 2 else p.normal_(1.0, 0.1)
    return c, m


def test_seq_cls_matches_transformers_and_roundtrips(tmp_path):
    from transformers import Qwen3ForSequenceClassification
    c, hf = _hf_base(Qwen3ForSequenceClassification)
    d1, d2 = str(tmp_path / 'a'), str(tmp_path / 'b')
    hf.save_pretrained(d1)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32, task_type='seq_cls', num_labels=3)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], d1)
    ids = torch.randint(1, 1024, (2, 32), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        per_token = model(ids)                                   # [b, s, num_labels]
        ref = hf(ids).logits                                     # [b, num_labels] taken at the last token
    assert per_token.shape == (2, 32, 3)
    assert torch.allclose(per_token[:, -1], ref, atol=1e-5)
    cfg.bridge.save_weights([model], d2)
    a, b = load_file(os.path.join(d1, 'model.safetensors')), load_file(os.path.join(d2, 'model.safetensors'))
    assert sorted(a) == sorted(b) and all(torch.equal(a[k], b[k]) for k in a)
    assert 'score.weight' in b


def test_embedding_and_reranker_heads(tmp_path):
    from transformers import Qwen3ForCausalLM
    c, hf = _hf_base(Qwen3ForCausalLM)
    d1 = str(tmp_path / 'a')
    hf.save_pretrained(d1)
    ids = torch.randint(1, 1024, (2, 16), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        out = hf(ids, output_hidden_states=True)
    # embedding: final-norm hidden states, L2 normalised
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32, task_type='embedding')
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], d1)
    with torch.no_grad():
        emb = model(ids)
    ref = torch.nn.functional.normalize(out.hidden_states[-1], dim=-1)
    assert torch.allclose(emb, ref, atol=1e-5)
    # generative reranker: logit(positive token) - logit(negative token)
    os.environ['GENERATIVE_RERANKER_POSITIVE_TOKEN_ID'] = '17'
    os.environ['GENERATIVE_RERANKER_NEGATIVE_TOKEN_ID'] = '900'
    try:
        cfg2 = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32, task_type='generative_reranker')
        model2 = get_mcore_model(cfg2)[0]
        cfg2.bridge.load_weights([model2], d1)
        with torch.no_grad():
            score = model2(ids)
        want = (out.logits[..., 17] - out.logits[..., 900]).unsqueeze(-1)
        assert torch.allclose(score, want, atol=1e-5)
    finally:
        os.environ.pop('GENERATIVE_RERANKER_POSITIVE_TOKEN_ID')
        os.environ.pop('GENERATIVE_RERANKER_NEGATIVE_TOKEN_ID')
