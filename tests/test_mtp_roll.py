import torch

from dist_utils import run_ranks
from mcore_bridge_b200.layers.context import PackedSeqParams
from mcore_bridge_b200.utils.megatron_utils import cp_gather_index, roll_tensor, split_cp_inputs


def test_roll_packed():
    t = torch.arange(1, 11).float()[None]
    psp = PackedSeqParams(cu_seqlens_q=torch.tensor([0, 4, 10], dtype=torch.int32))
    r, s = roll_tensor(t, -1, -1, None, psp)
    assert r.tolist() == [[2, 3, 4, 0, 6, 7, 8, 9, 10, 0]] and s.item() == r.sum().item()
    r2, _ = roll_tensor(t, -1, -1, None, None)
    assert r2.tolist() == [[2, 3, 4, 5, 6, 7, 8, 9, 10, 0]]


def test_split_and_gather_index():
    x = torch.arange(24)[None]
    cu = torch.tensor([0, 8, 24], dtype=torch.int32)
    parts = [split_cp_inputs(x, cu, -1, cp_size=2, cp_rank=r) for r in range(2)]
    assert parts[0].tolist() == [[0, 1, 6, 7, 8, 9, 10, 11, 20, 21, 22, 23]]
    assert parts[1].tolist() == [[2, 3, 4, 5, 12, 13, 14, 15, 16, 17, 18, 19]]
    idx = cp_gather_index(cu, 24, 2)
    assert torch.cat(parts, dim=-1)[0][idx].tolist() == list(range(24))


def _cp_worker(rank, world):
    import torch.distributed as dist

    from mcore_bridge_b200.parallel import state as ps
    ps.initialize_model_parallel(context_parallel_size=2)
    full = torch.arange(1, 25).float()[None]
    cu = torch.tensor([0, 8, 24], dtype=torch.int32)
    psp = PackedSeqParams(cu_seqlens_q=cu)
    local = split_cp_inputs(full, cu, -1)
    rolled, _ = roll_tensor(local, -1, -1, ps.get_group('cp'), psp)
    expect_full, _ = roll_tensor(full, -1, -1, None, psp)
    return torch.equal(rolled, split_cp_inputs(expect_full, cu, -1))


def test_roll_under_context_parallel():
    assert all(run_ranks(_cp_worker, 2))


def test_mtp_trains():
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    cfg = model_config('qwen3_tiny', params_dtype=torch.float32, mtp_num_layers=1)
    tr = Trainer(cfg, TrainConfig(lr=1e-3))
    ds = SyntheticPackedDataset(1024, 256, seg_lo=32, seg_hi=128)
    mbs = [ds.next_microbatch()]
    losses = [tr.train_step(mbs) for _ in range(4)]
    assert losses[-1] < losses[0]
    assert 'mtp_1_loss' in tr.last_metrics and tr.last_metrics['mtp_1_loss'] > 0
    mtp = tr.models[0].mtp.layers[0]
    assert mtp.eh_proj.weight.main_grad is not None
