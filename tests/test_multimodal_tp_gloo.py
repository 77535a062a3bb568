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
