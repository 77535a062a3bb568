"""Pipeline parallel (1F1B and virtual chunks) on gloo ranks reproduces the single-process training step."""
import torch

from dist_utils import run_ranks


def _run(rank, world, pp, vpp, tp, tied=False):
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                 virtual_pipeline_model_parallel_size=vpp)
    cfg = model_config('qwen3_tiny', {'tie_word_embeddings': True} if tied else None, params_dtype=torch.float32,
                       tensor_model_parallel_size=tp,
                       pipeline_model_parallel_size=pp, virtual_pipeline_model_parallel_size=vpp)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=0.0))
    # identical weights on every layout: fill each parameter from a generator seeded by its global name
    for m in tr.models:
        off = m.decoder.layer_offset
        for name, p in m.named_parameters():
            gname = name
            if name.startswith('decoder.layers.'):
                parts = name.split('.')
                parts[2] = str(int(parts[2]) + off)
                gname = '.'.join(parts)
            g = torch.Generator().manual_seed(abs(hash(gname)) % (2**31))
            full_shape = list(p.shape)
            with torch.no_grad():
                p.copy_(torch.randn(full_shape, generator=g) * 0.05 + (1.0 if p.dim() == 1 else 0.0))
    from mcore_bridge_b200.train.trainer import sync_shared_embeddings
    sync_shared_embeddings(tr.models)     # tied embeddings: the last stage's copy follows the first stage's
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, clip_grad=0.0)
    ds = SyntheticPackedDataset(1024, 256, seg_lo=32, seg_hi=128, seed=3)
    mbs = [ds.next_microbatch() for _ in range(4)]
    loss = tr.train_step(mbs)
    # collect a fingerprint of the updated weights by global name
    fp = {}
    for m in tr.models:
        off = m.decoder.layer_offset
        for name, p in m.named_parameters():
            if name.startswith('decoder.layers.'):
                parts = name.split('.')
                parts[2] = str(int(parts[2]) + off)
                name = '.'.join(parts)
            fp[name] = p.detach().double().sum().item()
    return loss, fp, ps.is_pipeline_last_stage()


def _hashseed_env():
    import os
    os.environ['PYTHONHASHSEED'] = '0'


def test_pp2_1f1b_matches_single():
    _hashseed_env()
    base = run_ranks(_run, 1, 1, None, 1)[0]
    res = run_ranks(_run, 2, 2, None, 1)
    last = [r for r in res if r[2]][0]
    assert abs(last[0] - base[0]) < 1e-5
    # every stage reports the step's loss, not only the last one
    assert all(abs(r[0] - base[0]) < 1e-5 for r in res), [r[0] for r in res]
    merged = {}
    for r in res:
        merged.update(r[1])
    for k, v in base[1].items():
        assert abs(merged[k] - v) < 1e-6 * max(1.0, abs(v)), k


def test_pp2_vpp2_matches_single():
    _hashseed_env()
    base = run_ranks(_run, 1, 1, None, 1)[0]
    res = run_ranks(_run, 2, 2, 2, 1)
    last = [r for r in res if r[2]][0]
    assert abs(last[0] - base[0]) < 1e-5
    merged = {}
    for r in res:
        merged.update(r[1])
    for k, v in base[1].items():
        assert abs(merged[k] - v) < 1e-6 * max(1.0, abs(v)), k


def test_pp2_tied_embeddings_match_single():
    """With tied input / output embeddings the two pipeline ends keep one copy each; their gradients are summed, so
    both copies end up equal to the single-process weight after the step."""
    _hashseed_env()
    base = run_ranks(_run, 1, 1, None, 1, True)[0]
    res = run_ranks(_run, 2, 2, None, 1, True)
    last = [r for r in res if r[2]][0]
    first = [r for r in res if not r[2]][0]
    assert abs(last[0] - base[0]) < 1e-5
    want = base[1]['embedding.word_embeddings.weight']
    assert 'output_layer.weight' not in base[1]
    assert abs(first[1]['embedding.word_embeddings.weight'] - want) < 1e-6 * max(1.0, abs(want))
    assert abs(last[1]['output_layer.weight'] - want) < 1e-6 * max(1.0, abs(want))
