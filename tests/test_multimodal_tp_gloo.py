"""Qwen3-VL with an image in the prompt on two tensor-parallel ranks (with and without sequence parallelism): loss and
the vision tower's gradients equal the single-process ones on every rank.  The tower is replicated; under sequence
parallelism each rank keeps the deepstack rows of its own tokens, so their gradients have to be summed over the group."""
import pytest
import torch

import test_multimodal_parity as MP
from dist_utils import run_ranks


def _worker(rank, world, ckpt, tp, sp):
    from transformers import AutoConfig

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    ps.initialize_model_parallel(tensor_model_parallel_size=tp)
    c = AutoConfig.from_pretrained(ckpt)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32, tensor_model_parallel_size=tp,
                      sequence_parallel=sp)
    model = get_mcore_model(cfg)[0].train()
    cfg.bridge.load_weights([model], ckpt)
    ids, pixels, grid = MP._inputs(c)
    labels = torch.randint(1, 400, ids.shape, generator=torch.Generator().manual_seed(5))
    loss = model(ids, position_ids=torch.load(ckpt + '/pos.pt'), labels=labels, pixel_values=pixels,
                 image_grid_thw=grid)
    loss.mean().backward()
    return loss.detach(), {n: p.grad.clone() for n, p in model.visual.named_parameters() if p.grad is not None}


@pytest.mark.parametrize('sp', [True, False])
def test_qwen3_vl_tower_gradients_tp2(tmp_path, sp):
    torch.manual_seed(0)
    c, hf = MP._qwen3_vl()
    hf = MP._randomise(hf.float().eval())
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    ids, _, grid = MP._inputs(c)
    pos, _ = hf.model.get_rope_index(ids, mm_token_type_ids=(ids == c.image_token_id).int(), image_grid_thw=grid)
    torch.save(pos, d + '/pos.pt')
    base_loss, base = run_ranks(_worker, 1, d, 1, False)[0]
    assert any('deepstack' in n for n in base)
    for loss, grads in run_ranks(_worker, 2, d, 2, sp):
        assert torch.allclose(loss, base_loss, atol=2e-5)
        for n, g in base.items():
            assert torch.allclose(grads[n], g, rtol=1e-4, atol=1e-6), (n, (grads[n] - g).abs().max().item())


def _train_worker(rank, world, ckpt, tp, pp):
    """Two optimizer steps through ``Trainer.train_step`` on micro-batches that carry an image (``pixel_values`` and
    ``image_grid_thw`` travel to the model as keyword arguments)."""
    from transformers import AutoConfig

    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp)
    c = AutoConfig.from_pretrained(ckpt)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32, tensor_model_parallel_size=tp,
                      pipeline_model_parallel_size=pp, sequence_parallel=tp > 1)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=1.0))
    cfg.bridge.load_weights(tr.models, ckpt)
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    ids, pixels, grid = MP._inputs(c)
    pos = torch.load(ckpt + '/pos.pt')
    losses = []
    for step in range(2):
        mbs = []
        for j in range(2):
            labels = torch.randint(1, 400, ids.shape, generator=torch.Generator().manual_seed(5 + 2 * step + j))
            mbs.append({'input_ids': ids, 'labels': labels, 'position_ids': pos, 'pixel_values': pixels,
                        'image_grid_thw': grid})
        losses.append(tr.train_step(mbs))
    return losses, {k: v.clone() for k, v in cfg.bridge.export_weights(tr.models)}, ps.is_pipeline_last_stage()


def test_qwen2_5_vl_trains_through_the_trainer_tp2_pp2(tmp_path):
    torch.manual_seed(0)
    c, hf = MP._qwen2_5_vl()
    hf = MP._randomise(hf.float().eval())
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    ids, _, grid = MP._inputs(c)
    pos, _ = hf.model.get_rope_index(ids, mm_token_type_ids=(ids == c.image_token_id).int(), image_grid_thw=grid)
    torch.save(pos, d + '/pos.pt')
    base_losses, base_w, _ = run_ranks(_train_worker, 1, d, 1, 1)[0]
    tower = [k for k in base_w if 'visual' in k]
    assert tower
    # the tower was trained: its weights moved away from the checkpoint
    from safetensors.torch import load_file
    start = load_file(d + '/model.safetensors')
    assert any(not torch.equal(base_w[k], start[k]) for k in tower if k in start)
    for losses, w, last in run_ranks(_train_worker, 4, d, 2, 2):
        if last:
            for a, b in zip(losses, base_losses):
                assert abs(a - b) < 3e-5, (losses, base_losses)
        assert set(w) == set(base_w)
        for k, v in base_w.items():
            assert torch.allclose(w[k], v, rtol=0, atol=3e-6), (k, (w[k] - v).abs().max().item())
