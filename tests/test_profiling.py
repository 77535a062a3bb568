"""Tracing helpers: NVTX ranges are a shared do-nothing object unless tracing is on and CUDA is present; the device
timers are inert without CUDA; a trainer with ``device_timers`` still steps on CPU."""
import torch


def test_ranges_and_timers_are_inert_without_cuda():
    from mcore_bridge_b200.utils import profiling
    a, b = profiling.nvtx_range('qkv'), profiling.nvtx_range('core_attention')
    assert a is b
    with a:
        pass
    profiling.set_nvtx(True)
    try:
        if not torch.cuda.is_available():
            assert profiling.nvtx_range('x') is a
    finally:
        profiling.set_nvtx(False)
    t = profiling.DeviceTimers()
    with t.time('optimizer'):
        pass
    if not torch.cuda.is_available():
        assert t.summary() == {}


def test_trainer_with_device_timers_steps_on_cpu():
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel()
    cfg = model_config('qwen3_tiny')
    tr = Trainer(cfg, TrainConfig(lr=1e-3, device_timers=True))
    ds = SyntheticPackedDataset(cfg.padded_vocab_size, 128, seg_lo=32, seg_hi=64, seed=1, pin=False)
    loss = tr.train_step([ds.next_microbatch()])
    assert loss > 0 and 'loss' in tr.last_metrics
    if torch.cuda.is_available():
        assert tr.last_metrics['forward_backward_ms'] > 0 and tr.last_metrics['optimizer_ms'] > 0
