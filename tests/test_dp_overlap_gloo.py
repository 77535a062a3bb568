"""Data parallel over 2 gloo ranks: the bucketed gradient reduction that overlaps with backward must give exactly the
result of reducing after backward, and every parameter must report its gradient exactly once per backward pass (a
weight whose backward writes straight into ``main_grad`` is also visited by autograd's accumulate node, which must
not report it a second time: the bucket would be reduced before the gradients produced later exist)."""
import pytest
import torch

from dist_utils import run_ranks


def _worker(rank, world, tied):
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel()
    out = {}
    for overlap in (True, False):
        torch.manual_seed(0)
        cfg = model_config('qwen3_tiny', untie_embeddings_and_output_weights=not tied)
        tr = Trainer(cfg, TrainConfig(lr=1e-3, overlap_grad_reduce=overlap))
        calls = {}
        for m in tr.ddp:
            for buf in m.buffers.values():
                for p in buf.params:
                    def counted(orig=p.grad_ready_hook, p=p, m=m):
                        if m.is_last_microbatch:
                            calls[id(p)] = calls.get(id(p), 0) + 1
                        orig()
                    p.grad_ready_hook = counted
        ds = SyntheticPackedDataset(cfg.padded_vocab_size, 256, seg_lo=32, seg_hi=128, seed=11 + rank, pin=False)
        loss = tr.train_step([ds.next_microbatch() for _ in range(2)])
        names = {id(p): n for m in tr.models for n, p in m.named_parameters()}
        expect = {id(p): int(getattr(p, 'grad_contributions', 1)) for m in tr.models for p in m.parameters()}
        wrong = {names[k]: (calls.get(k, 0), v) for k, v in expect.items() if calls.get(k, 0) != v}
        flat = torch.cat([p.detach().float().reshape(-1) for m in tr.models for p in m.parameters()])
        out[overlap] = (loss, flat, wrong)
    return out[True][0], out[False][0], torch.equal(out[True][1], out[False][1]), out[True][2], out[True][1]


@pytest.mark.parametrize('tied', [False, True])
def test_overlapped_reduction_equals_reduction_after_backward(tied):
    res = run_ranks(_worker, 2, tied)
    for loss_a, loss_b, same, wrong, _ in res:
        assert not wrong, f'parameters reporting a wrong number of times (got, expected): {wrong}'
        assert loss_a == loss_b
        assert same, 'overlapped and deferred gradient reduction gave different parameters after one step'
    assert torch.equal(res[0][4], res[1][4]), 'data-parallel ranks hold different parameters after one step'


def _gather_worker(rank, world):
    """Three steps with the parameter all-gather overlapped with the next forward pass against three steps with the
    all-gather inside ``step``; small buckets so that every layer waits for buckets of its own."""
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel()
    out = {}
    for overlap in (True, False):
        torch.manual_seed(0)
        cfg = model_config('qwen3_moe_tiny')
        tr = Trainer(cfg, TrainConfig(lr=1e-3, bucket_mb=0.05, overlap_param_gather=overlap))
        ds = SyntheticPackedDataset(cfg.padded_vocab_size, 256, seg_lo=32, seg_hi=128, seed=11 + rank, pin=False)
        losses, in_flight = [], []
        for _ in range(3):
            losses.append(tr.train_step([ds.next_microbatch() for _ in range(2)]))
            in_flight.append(len(tr.optimizer._pending))
        n_buckets = sum(len(buf.buckets) for m in tr.ddp for buf in m.buffers.values())
        sd = tr.optimizer.state_dict()                       # waits for what is in flight
        assert not tr.optimizer._pending and sd['step'] == 3
        flat = torch.cat([p.detach().float().reshape(-1) for m in tr.models for p in m.parameters()])
        out[overlap] = (losses, flat, in_flight, n_buckets)
    return out


def test_overlapped_parameter_gather_equals_gather_inside_the_step():
    res = run_ranks(_gather_worker, 2)
    for out in res:
        (la, pa, fa, nb), (lb, pb, fb, _) = out[True], out[False]
        assert la == lb and torch.equal(pa, pb)
        assert fb == [0, 0, 0] and fa == [nb, nb, nb] and nb > 4       # every bucket was left in flight by the step
    assert torch.equal(res[0][True][1], res[1][True][1]), 'data-parallel ranks hold different parameters'


def _export_worker(rank, world):
    """The checkpoint bridge reads parameters without running the model: with the all-gather still in flight it has to
    wait for it itself."""
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel()
    out = {}
    for overlap in (True, False):
        torch.manual_seed(0)
        cfg = model_config('qwen3_tiny')
        tr = Trainer(cfg, TrainConfig(lr=1e-3, bucket_mb=0.05, overlap_param_gather=overlap))
        ds = SyntheticPackedDataset(cfg.padded_vocab_size, 256, seg_lo=32, seg_hi=128, seed=11 + rank, pin=False)
        tr.train_step([ds.next_microbatch() for _ in range(2)])
        pending = len(tr.optimizer._pending)
        out[overlap] = ({k: v.clone() for k, v in cfg.bridge.export_weights(tr.models)}, pending)
    return out


def test_export_waits_for_the_overlapped_gather():
    for out in run_ranks(_export_worker, 2):
        (wa, pa), (wb, pb) = out[True], out[False]
        assert pa > 0 and pb == 0
        assert wa.keys() == wb.keys() and all(torch.equal(wa[k], wb[k]) for k in wa)
