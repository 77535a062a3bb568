"""Two optimizer steps on four gloo ranks — tensor x data parallel (with sequence parallelism) for a dense model,
expert x data parallel for an MoE model — against the same two steps in one process: losses and every exported weight
must agree.  Weights travel through the Hugging Face checkpoint bridge, so every layout starts from identical values;
the global batch is the same four micro-batches, dealt out to the data-parallel ranks."""
import torch

from dist_utils import run_ranks

STEPS, GLOBAL_MB = 2, 4
_BASE = {}      # single-process results, shared by the layouts of one model / loss configuration


def _worker(rank, world, name, ckpt, tp, ep, aux, pp=1, cp=1, etp=1, hf_over=None, over=None):
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=etp, pipeline_model_parallel_size=pp,
                                 context_parallel_size=cp)
    extra = dict(moe_aux_loss_coeff=aux) if aux else {}
    extra.update(over or {})
    cfg = model_config(name, hf_over, params_dtype=torch.float32, tensor_model_parallel_size=tp,
                       expert_model_parallel_size=ep, expert_tensor_parallel_size=etp,
                       pipeline_model_parallel_size=pp, context_parallel_size=cp,
                       sequence_parallel=tp > 1, **extra)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=1.0))
    cfg.bridge.load_weights(tr.models, ckpt)
    # master weights from the loaded values; a large epsilon keeps Adam's step a smooth function of the gradient, so
    # layouts that differ only in summation order stay within rounding of each other
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    dp, dp_rank = ps.get_world_size('dp'), ps.get_rank_in('dp') if ps.get_world_size('dp') > 1 else 0
    # segment lengths in multiples of 4 so that the zig-zag context-parallel split (2 * cp chunks) applies
    ds = SyntheticPackedDataset(1024, 256, seg_lo=32, seg_hi=128, seed=3, pin=False, segment_multiple=4)
    losses = []
    for _ in range(STEPS):
        mbs = [ds.next_microbatch() for _ in range(GLOBAL_MB)]
        losses.append(tr.train_step(mbs[dp_rank::dp]))
    weights = {k: v.clone() for k, v in cfg.bridge.export_weights(tr.models)}
    return losses, weights, ps.is_pipeline_last_stage()


def _check(tmp_path, name, hf_cls, tp, ep, aux=0.0, pp=1, cp=1, etp=1, hf_over=None, over=None):
    from mcore_bridge_b200.train.presets import hf_config
    torch.manual_seed(0)
    hf = hf_cls(hf_config(name, **(hf_over or {}))).float()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0, 0.05)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    key = (name, aux, repr(sorted((hf_over or {}).items())), repr(sorted((over or {}).items())))
    if key not in _BASE:        # the checkpoint is a function of the key (seeded), so the reference run is too
        _BASE[key] = run_ranks(_worker, 1, name, d, 1, 1, aux, 1, 1, 1, hf_over, over)[0]
    base_losses, base_w, _ = _BASE[key]
    res = run_ranks(_worker, 4, name, d, tp, ep, aux, pp, cp, etp, hf_over, over)
    for losses, weights, last_stage in res:
        if last_stage:                      # only the last pipeline stage sees the loss
            for a, b in zip(losses, base_losses):
                assert abs(a - b) < 2e-5, (losses, base_losses)
        assert set(weights) == set(base_w)
        for k, v in base_w.items():
            assert torch.allclose(weights[k], v, rtol=0, atol=2e-6), (k, (weights[k] - v).abs().max().item())


def test_dense_tp2_dp2_matches_single_process(tmp_path):
    from transformers import Qwen3ForCausalLM
    _check(tmp_path, 'qwen3_tiny', Qwen3ForCausalLM, tp=2, ep=1)


def test_moe_ep2_dp_matches_single_process(tmp_path):
    from transformers import Qwen3MoeForCausalLM
    _check(tmp_path, 'qwen3_moe_tiny', Qwen3MoeForCausalLM, tp=1, ep=2, aux=1e-2)


def test_dense_pp2_dp2_matches_single_process(tmp_path):
    from transformers import Qwen3ForCausalLM
    _check(tmp_path, 'qwen3_tiny', Qwen3ForCausalLM, tp=1, ep=1, pp=2)


def test_dense_cp2_dp2_matches_single_process(tmp_path):
    from transformers import Qwen3ForCausalLM
    _check(tmp_path, 'qwen3_tiny', Qwen3ForCausalLM, tp=1, ep=1, cp=2)


def test_moe_tp2_ep2_matches_single_process(tmp_path):
    from transformers import Qwen3MoeForCausalLM
    _check(tmp_path, 'qwen3_moe_tiny', Qwen3MoeForCausalLM, tp=2, ep=2, aux=1e-2)


def test_dense_tp2_pp2_matches_single_process(tmp_path):
    from transformers import Qwen3ForCausalLM
    _check(tmp_path, 'qwen3_tiny', Qwen3ForCausalLM, tp=2, ep=1, pp=2)


def test_moe_expert_tensor_parallel_dp2_matches_single_process(tmp_path):
    from transformers import Qwen3MoeForCausalLM
    _check(tmp_path, 'qwen3_moe_tiny', Qwen3MoeForCausalLM, tp=2, ep=1, etp=2, aux=1e-2)


def test_moe_ep2_pp2_matches_single_process(tmp_path):
    from transformers import Qwen3MoeForCausalLM
    _check(tmp_path, 'qwen3_moe_tiny', Qwen3MoeForCausalLM, tp=1, ep=2, pp=2, aux=1e-2)


def test_moe_seq_aux_loss_tp2_ep2_matches_single_process(tmp_path):
    from transformers import Qwen3MoeForCausalLM
    _check(tmp_path, 'qwen3_moe_tiny', Qwen3MoeForCausalLM, tp=2, ep=2, aux=1e-2,
           over={'moe_router_load_balancing_type': 'seq_aux_loss'})


def test_dense_tied_embeddings_pp2_dp2_matches_single_process(tmp_path):
    """The tied matrix lives on both pipeline ends; its gradient is summed over the two copies and must enter the
    clipping norm once."""
    from transformers import Qwen3ForCausalLM
    _check(tmp_path, 'qwen3_tiny', Qwen3ForCausalLM, tp=1, ep=1, pp=2, hf_over={'tie_word_embeddings': True})


def test_moe_z_loss_tp2_ep2_matches_single_process(tmp_path):
    """The router z-loss is a mean over tokens: with the tokens split over the tensor-parallel ranks (sequence
    parallelism) every rank adds its share of it."""
    from transformers import Qwen3MoeForCausalLM
    _check(tmp_path, 'qwen3_moe_tiny', Qwen3MoeForCausalLM, tp=2, ep=2, aux=1e-2, over={'moe_z_loss_coeff': 1e-2})
