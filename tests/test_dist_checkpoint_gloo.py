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
