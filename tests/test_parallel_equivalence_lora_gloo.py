"""LoRA fine-tuning in different layouts: two optimizer steps of the adapters (dense and grouped-expert LoRA, frozen
base) on four gloo ranks against one process.  Base weights and the initial adapter travel through the checkpoint
bridge (Hugging Face and PEFT formats), the trained adapters are compared in PEFT format."""
import torch

from dist_utils import run_ranks

STEPS, GLOBAL_MB = 2, 4


def _worker(rank, world, name, ckpt, adapter, tp, ep, save_to=None):
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=1)
    cfg = model_config(name, params_dtype=torch.float32, tensor_model_parallel_size=tp,
                       expert_model_parallel_size=ep, expert_tensor_parallel_size=1, sequence_parallel=tp > 1)
    models = get_mcore_model(cfg)
    cfg.bridge.load_weights(models, ckpt)
    models = [get_peft_model(m, LoraConfig(r=8, lora_alpha=16, target_modules='all-linear')) for m in models]
    if adapter is None:             # first call: make a non-trivial adapter and publish it
        g = torch.Generator().manual_seed(3)
        with torch.no_grad():
            for m in models:
                for n, p in m.named_parameters():
                    if 'lora_' in n:
                        p.copy_(torch.randn(p.shape, generator=g) * 0.05)
        cfg.bridge.save_weights(models, save_to, peft_format=True)
        return None
    cfg.bridge.load_weights(models, adapter, peft_format=True)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=1.0), models=models)
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    dp, dp_rank = ps.get_world_size('dp'), ps.get_rank_in('dp') if ps.get_world_size('dp') > 1 else 0
    ds = SyntheticPackedDataset(1024, 256, seg_lo=32, seg_hi=128, seed=3, pin=False, segment_multiple=4)
    losses = []
    for _ in range(STEPS):
        mbs = [ds.next_microbatch() for _ in range(GLOBAL_MB)]
        losses.append(tr.train_step(mbs[dp_rank::dp]))
    weights = {k: v.clone() for k, v in cfg.bridge.export_weights(tr.models, peft_format=True)}
    return losses, weights


def _check(tmp_path, name, hf_cls, tp, ep):
    from mcore_bridge_b200.train.presets import hf_config
    torch.manual_seed(0)
    hf = hf_cls(hf_config(name)).float()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0, 0.05)
    d, a = str(tmp_path / 'ckpt'), str(tmp_path / 'adapter')
    hf.save_pretrained(d)
    run_ranks(_worker, 1, name, d, None, 1, 1, a)
    base_losses, base_w = run_ranks(_worker, 1, name, d, a, 1, 1)[0]
    assert any('lora_B' in k for k in base_w)
    for losses, weights in run_ranks(_worker, 4, name, d, a, tp, ep):
        for x, y in zip(losses, base_losses):
            assert abs(x - y) < 2e-5, (losses, base_losses)
        assert set(weights) == set(base_w)
        for k, v in base_w.items():
            assert torch.allclose(weights[k], v, rtol=0, atol=2e-6), (k, (weights[k] - v).abs().max().item())


def test_lora_dense_tp2_dp2_matches_single_process(tmp_path):
    from transformers import Qwen3ForCausalLM
    _check(tmp_path, 'qwen3_tiny', Qwen3ForCausalLM, tp=2, ep=1)


def test_lora_moe_tp2_ep2_matches_single_process(tmp_path):
    from transformers import Qwen3MoeForCausalLM
    _check(tmp_path, 'qwen3_moe_tiny', Qwen3MoeForCausalLM, tp=2, ep=2)


# ------------------------------------------------------------------ MLA families: adapters on replicated projections
def _family_worker(rank, world, ckpt, adapter, tp, ep, save_to=None):
    from transformers import AutoConfig

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=1)
    cfg = ModelConfig(**hf_to_mcore_config(AutoConfig.from_pretrained(ckpt)), params_dtype=torch.float32,
                      tensor_model_parallel_size=tp, expert_model_parallel_size=ep, expert_tensor_parallel_size=1,
                      sequence_parallel=tp > 1)
    models = get_mcore_model(cfg)
    cfg.bridge.load_weights(models, ckpt)
    models = [get_peft_model(m, LoraConfig(r=4, lora_alpha=8, target_modules='all-linear')) for m in models]
    if adapter is None:
        g = torch.Generator().manual_seed(3)
        with torch.no_grad():
            for m in models:
                for n, p in sorted(m.named_parameters(), key=lambda kv: kv[0]):
                    if 'lora_' in n:
                        p.copy_(torch.randn(p.shape, generator=g) * 0.05)
        cfg.bridge.save_weights(models, save_to, peft_format=True)
        return None
    cfg.bridge.load_weights(models, adapter, peft_format=True)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=1.0), models=models)
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    dp, dp_rank = ps.get_world_size('dp'), ps.get_rank_in('dp') if ps.get_world_size('dp') > 1 else 0
    ds = SyntheticPackedDataset(256, 256, seg_lo=32, seg_hi=128, seed=3, pin=False, segment_multiple=4)
    losses = []
    for _ in range(STEPS):
        mbs = [ds.next_microbatch() for _ in range(GLOBAL_MB)]
        losses.append(tr.train_step(mbs[dp_rank::dp]))
    return losses, {k: v.clone() for k, v in cfg.bridge.export_weights(tr.models, peft_format=True)}


def _check_family(tmp_path, hf, tp, ep, expect_keys):
    torch.manual_seed(0)
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0 if 'norm' in n else 0.0, 0.05)
    d, a = str(tmp_path / 'ckpt'), str(tmp_path / 'adapter')
    hf.save_pretrained(d)
    run_ranks(_family_worker, 1, d, None, 1, 1, a)
    base_losses, base_w = run_ranks(_family_worker, 1, d, a, 1, 1)[0]
    for frag in expect_keys:
        assert any(frag in k for k in base_w), frag
    for losses, weights in run_ranks(_family_worker, 4, d, a, tp, ep):
        for x, y in zip(losses, base_losses):
            assert abs(x - y) < 3e-5, (losses, base_losses)
        assert set(weights) == set(base_w)
        for k, v in base_w.items():
            assert torch.allclose(weights[k], v, rtol=0, atol=2e-6), (k, (weights[k] - v).abs().max().item())
    return base_w


def test_lora_glm_dsa_tp2_ep2_matches_single_process(tmp_path):
    """MLA with a query low-rank path and the DSA indexer: adapters on the replicated down projections (run on this
    rank's tokens under sequence parallelism, no collective of their own), on the fused norm + up projections (whose
    normalised input also feeds the indexer) and on the indexer's linears."""
    import test_parallel_equivalence_families_gloo as Fm
    _check_family(tmp_path, Fm._glm_dsa(), 2, 2, ['q_a_proj.lora_B', 'indexer.wq_b.lora_A'])


def test_lora_gemma4_tp2_dp2_matches_single_process(tmp_path):
    """Gemma-4: per-layer-type head sizes and KV head counts in the packed q / k / v adapter, layers without a value
    projection (k = v) or without keys and values of their own (shared KV), the per-layer-input projections (one of
    them a model-level column-parallel linear that hands out its gathered output) and the MoE branch."""
    import test_parallel_equivalence_families_gloo as Fm
    w = _check_family(tmp_path, Fm._gemma4(), 2, 1,
                      ['layers.0.self_attn.v_proj.lora_B', 'layers.2.self_attn.k_proj.lora_B',
                       'per_layer_model_projection.lora_A', 'layers.0.per_layer_input_gate.lora_B',
                       'layers.0.experts.1.gate_proj.lora_B'])
    assert not any('layers.2.self_attn.v_proj' in k for k in w)         # full-attention layers: k = v
    assert not any('layers.5.self_attn.k_proj' in k for k in w)         # shared-KV tail layers project queries only
