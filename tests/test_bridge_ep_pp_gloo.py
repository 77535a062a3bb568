"""Bridge under expert and pipeline parallelism (gloo): a Qwen3-MoE checkpoint loaded on EP=2 / PP=2 layouts gives the
Transformers loss and exports, on every rank, exactly the tensors it was loaded from."""
import torch

from dist_utils import run_ranks


def _setup(tmp):
    from transformers import Qwen3MoeForCausalLM

    from mcore_bridge_b200.train.presets import hf_config
    torch.manual_seed(0)
    c = hf_config('qwen3_moe_tiny')
    hf = Qwen3MoeForCausalLM(c).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.02) if p.dim() >= 2 else p.normal_(1.0, 0.1)
    hf.save_pretrained(tmp)
    return c, hf


def _batch():
    g = torch.Generator().manual_seed(1)
    return torch.randint(0, 1024, (2, 64), generator=g), torch.randint(0, 1024, (2, 64), generator=g)


def _worker(rank, world, ckpt, ep, pp):
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.presets import hf_config
    ps.initialize_model_parallel(expert_model_parallel_size=ep, pipeline_model_parallel_size=pp)
    cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_moe_tiny')), params_dtype=torch.float32,
                      expert_model_parallel_size=ep, pipeline_model_parallel_size=pp)
    models = get_mcore_model(cfg)
    cfg.bridge.load_weights(models, ckpt)
    exported = {k: v.clone() for k, v in cfg.bridge.export_weights(models)}
    loss = None
    if pp == 1:
        ids, labels = _batch()
        half = slice(rank, rank + 1)          # EP ranks are data-parallel for the dense part: one sample each
        loss = models[0](ids[half], labels=labels[half]).detach()
    return exported, loss


def _check(tmp_path, ep, pp):
    d = str(tmp_path / 'ckpt')
    c, hf = _setup(d)
    res = run_ranks(_worker, ep * pp, d, ep, pp)
    import os

    from safetensors.torch import load_file
    sd = load_file(os.path.join(d, 'model.safetensors'))      # the on-disk layout (per-expert keys)
    for exported, _ in res:
        assert sorted(exported) == sorted(sd)
        for k, v in exported.items():
            assert torch.equal(v, sd[k]), k
    if pp == 1:
        ids, labels = _batch()
        with torch.no_grad():
            logits = hf(ids).logits
        ref = torch.nn.functional.cross_entropy(logits.view(-1, 1024), labels.view(-1), reduction='none').view(2, 64)
        for r, (_, loss) in enumerate(res):
            assert torch.allclose(loss[0], ref[r], atol=2e-5)


def test_bridge_ep2(tmp_path):
    _check(tmp_path, 2, 1)


def test_bridge_pp2(tmp_path):
    _check(tmp_path, 1, 2)
