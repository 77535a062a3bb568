"""Sharded checkpoints are layout independent: saved on four ranks under one layout, loaded under another (and in one
process), the models export identical Hugging Face weights."""
import torch

from dist_utils import run_ranks


def _worker(rank, world, name, tp, pp, ep, directory, mode, seed):
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train import dist_checkpoint as dc
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import init_weights
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                 expert_model_parallel_size=ep, expert_tensor_parallel_size=1)
    cfg = model_config(name, params_dtype=torch.float32, tensor_model_parallel_size=tp,
                       pipeline_model_parallel_size=pp, expert_model_parallel_size=ep, expert_tensor_parallel_size=1,
                       sequence_parallel=tp > 1)
    models = get_mcore_model(cfg)
    if mode == 'save':
        # identical full weights whatever the layout: fill from a Hugging Face state dict made with one seed
        from mcore_bridge_b200.utils.safetensors import LazyTensor
        full = torch.load(seed)
        for _ in cfg.bridge._convert(models, {k: LazyTensor(tensor=v) for k, v in full.items()}, True):
            pass
        dc.save(models, directory)
    else:
        for m in models:
            init_weights(m, 0.3, 99 + rank)          # garbage that the load has to replace completely
        dc.load(models, directory)
    return {k: v.clone() for k, v in cfg.bridge.export_weights(models)}


def _check(tmp_path, name, save_layout, load_layouts):
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import init_weights
    cfg = model_config(name, params_dtype=torch.float32)
    m = get_mcore_model(cfg)[0]
    init_weights(m, 0.05, 7)
    ref = dict(cfg.bridge.export_weights([m]))
    seed = str(tmp_path / 'full.pt')
    torch.save(ref, seed)
    d = str(tmp_path / 'ckpt')
    world, tp, pp, ep = save_layout
    run_ranks(_worker, world, name, tp, pp, ep, d, 'save', seed)
    for world, tp, pp, ep in load_layouts:
        for exported in run_ranks(_worker, world, name, tp, pp, ep, d, 'load', seed):
            assert set(exported) == set(ref)
            for k, v in ref.items():
                assert torch.equal(exported[k], v), (k, (world, tp, pp, ep))


def test_dense_tp2_pp2_to_other_layouts(tmp_path):
    _check(tmp_path, 'qwen3_tiny', (4, 2, 2, 1), [(1, 1, 1, 1), (2, 2, 1, 1), (2, 1, 2, 1)])


def test_moe_tp2_ep2_to_other_layouts(tmp_path):
    _check(tmp_path, 'qwen3_moe_tiny', (4, 2, 1, 2), [(1, 1, 1, 1), (2, 1, 1, 2)])


def _lora_worker(rank, world, tp, pp, directory, mode, adapter):
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train import dist_checkpoint as dc
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import init_weights
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp)
    cfg = model_config('qwen3_tiny', params_dtype=torch.float32, tensor_model_parallel_size=tp,
                       pipeline_model_parallel_size=pp, sequence_parallel=tp > 1)
    models = get_mcore_model(cfg)
    for m in models:
        init_weights(m, 0.05, 7)
    models = [get_peft_model(m, LoraConfig(r=4, lora_alpha=8, target_modules='all-linear')) for m in models]
    if mode == 'save':
        cfg.bridge.load_weights(models, adapter, peft_format=True)
        dc.save(models, directory)
    else:
        with torch.no_grad():
            for m in models:
                for n, p in m.named_parameters():
                    if 'lora_' in n:
                        p.normal_(0, 0.3)               # garbage that the load has to replace
        dc.load(models, directory)
    return {k: v.clone() for k, v in cfg.bridge.export_weights(models, peft_format=True)}


def test_lora_adapters_reshard(tmp_path):
    """Adapter factors follow the layout of the linear they sit on: ``lora_B`` of a gated MLP keeps [gate shard; up
    shard] on every rank and is re-partitioned with that stride."""
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    cfg = model_config('qwen3_tiny', params_dtype=torch.float32)
    peft = get_peft_model(get_mcore_model(cfg)[0], LoraConfig(r=4, lora_alpha=8, target_modules='all-linear'))
    g = torch.Generator().manual_seed(7)
    with torch.no_grad():
        for n, p in sorted(peft.named_parameters(), key=lambda kv: kv[0]):
            if 'lora_' in n:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    adapter = str(tmp_path / 'adapter')
    cfg.bridge.save_weights([peft], adapter, peft_format=True)
    ref = dict(cfg.bridge.export_weights([peft], peft_format=True))
    d = str(tmp_path / 'ckpt')
    run_ranks(_lora_worker, 4, 2, 2, d, 'save', adapter)
    for world, tp, pp in [(1, 1, 1), (2, 2, 1)]:
        for exported in run_ranks(_lora_worker, world, tp, pp, d, 'load', adapter):
            assert set(exported) == set(ref)
            for k, v in ref.items():
                assert torch.equal(exported[k], v), (k, (world, tp, pp))
