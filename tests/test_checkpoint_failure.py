"""Checkpoint/resume of the training state, corruption detection, and host-side failure detection (a rank that never
joins a collective ends the others' wait with an error inside the process-group timeout)."""
import json
import os

import pytest
import torch

from dist_utils import run_ranks


def _trainer():
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    cfg = model_config('qwen3_tiny', params_dtype=torch.float32)
    return Trainer(cfg, TrainConfig(lr=1e-3, init_seed=7))


def test_resume_reproduces_next_step(tmp_path):
    from mcore_bridge_b200.train.checkpoint import load_training_state, save_training_state
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    ds = SyntheticPackedDataset(1024, 256, seg_lo=32, seg_hi=128, seed=1)
    mbs = [ds.next_microbatch() for _ in range(3)]
    a = _trainer()
    a.train_step(mbs[:1])
    a.train_step(mbs[1:2])
    d_model, d_state = str(tmp_path / 'model'), str(tmp_path / 'state')
    a.config.bridge.save_weights(a.models, d_model)
    save_training_state(a, d_state, step=2, extra={'consumed': 2})
    loss_a = a.train_step(mbs[2:3])
    b = _trainer()
    b.config.bridge.load_weights(b.models, d_model)
    m = load_training_state(b, d_state)
    assert m['step'] == 2 and m['extra']['consumed'] == 2 and b.optimizer.step_count == 2
    loss_b = b.train_step(mbs[2:3])
    assert abs(loss_a - loss_b) < 1e-5
    for pa, pb in zip(a.models[0].parameters(), b.models[0].parameters()):
        assert torch.allclose(pa, pb, atol=1e-6)


def test_corrupt_shard_and_missing_manifest_are_detected(tmp_path):
    from mcore_bridge_b200.train.checkpoint import load_training_state, save_training_state
    a = _trainer()
    d = str(tmp_path / 'state')
    save_training_state(a, d, step=0)
    path = os.path.join(d, 'optim_rank00000.safetensors')
    raw = bytearray(open(path, 'rb').read())
    raw[-1] ^= 0xFF
    open(path, 'wb').write(bytes(raw))
    with pytest.raises(IOError):
        load_training_state(a, d)
    os.remove(os.path.join(d, 'manifest.json'))
    with pytest.raises(FileNotFoundError):
        load_training_state(a, d)


def test_layout_mismatch_refused(tmp_path):
    from mcore_bridge_b200.train.checkpoint import load_training_state, save_training_state
    a = _trainer()
    d = str(tmp_path / 'state')
    save_training_state(a, d, step=0)
    m = json.load(open(os.path.join(d, 'manifest.json')))
    m['layout']['tp'] = 2
    json.dump(m, open(os.path.join(d, 'manifest.json'), 'w'))
    with pytest.raises(ValueError):
        load_training_state(a, d)


def _absent_rank(rank, world):
    """Rank 1 leaves between steps without joining the next collective; rank 0 must get an error, not hang."""
    import time
    from datetime import timedelta

    import torch.distributed as dist
    g = dist.new_group([0, 1], backend='gloo', timeout=timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t, group=g)          # step 1: both present
    if rank == 1:
        return 'left'
    t0 = time.time()
    try:
        dist.all_reduce(t, group=g)      # step 2: the peer is gone
        return 'no error'
    except Exception as e:
        return f'detected after {time.time() - t0:.1f}s: {type(e).__name__}'


def test_missing_rank_is_detected_by_timeout():
    res = run_ranks(_absent_rank, 2, timeout=60)
    assert res[1] == 'left'
    assert res[0].startswith('detected'), res[0]


def test_heartbeat_store_flags_dead_rank(tmp_path):
    """Ranks publish a heartbeat in a store between steps; a monitor sees which rank stopped."""
    from mcore_bridge_b200.train.health import HeartbeatMonitor
    path = str(tmp_path / 'hb')
    mons = [HeartbeatMonitor(path, rank=r, world=3, timeout_s=0.5) for r in range(3)]
    for m in mons:
        m.beat(step=1)
    assert mons[0].dead_ranks() == []
    import time
    time.sleep(0.7)
    mons[0].beat(step=2)
    mons[2].beat(step=2)
    assert mons[0].dead_ranks() == [1]
