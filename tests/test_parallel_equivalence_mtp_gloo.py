"""Multi-token prediction in different layouts: a tiny DeepSeek-V3-style model with one MTP depth, two optimizer steps
on four gloo ranks against one process.  The starting checkpoint (MTP layer included) is written by the bridge from a
seeded single-process model, then loaded by every layout."""
import torch

from dist_utils import run_ranks

STEPS, GLOBAL_MB = 2, 4


def _config():
    from transformers import DeepseekV3Config
    return DeepseekV3Config(num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                            q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                            n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
                            moe_intermediate_size=32, intermediate_size=128, first_k_dense_replace=1,
                            n_shared_experts=1, vocab_size=256, max_position_embeddings=512,
                            tie_word_embeddings=False, num_nextn_predict_layers=1)


def _worker(rank, world, ckpt, tp, ep, cp, make, pp=1, tied=False):
    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=1, context_parallel_size=cp,
                                 pipeline_model_parallel_size=pp)
    kw = hf_to_mcore_config(_config())
    kw.update(mtp_num_layers=1, moe_aux_loss_coeff=1e-2)
    if tied:
        kw['untie_embeddings_and_output_weights'] = False
    cfg = ModelConfig(**kw, params_dtype=torch.float32, tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                      expert_tensor_parallel_size=1, context_parallel_size=cp, pipeline_model_parallel_size=pp,
                      sequence_parallel=tp > 1)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=7, clip_grad=1.0))
    if make:
        cfg.bridge.save_weights(tr.models, ckpt)
        return None
    cfg.bridge.load_weights(tr.models, ckpt)
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    dp, dp_rank = ps.get_world_size('dp'), ps.get_rank_in('dp') if ps.get_world_size('dp') > 1 else 0
    ds = SyntheticPackedDataset(256, 256, seg_lo=32, seg_hi=128, seed=3, pin=False, segment_multiple=4)
    losses = []
    for _ in range(STEPS):
        mbs = [ds.next_microbatch() for _ in range(GLOBAL_MB)]
        losses.append((tr.train_step(mbs[dp_rank::dp]), tr.last_metrics.get('mtp_1_loss')))
    weights = {k: v.clone() for k, v in cfg.bridge.export_weights(tr.models)}
    return losses, weights


def _check(tmp_path, layouts, tied=False):
    d = str(tmp_path / 'ckpt')
    run_ranks(_worker, 1, d, 1, 1, 1, True, 1, tied)
    base_losses, base_w = run_ranks(_worker, 1, d, 1, 1, 1, False, 1, tied)[0]
    assert base_losses[0][1] is not None and any('layers.2.' in k for k in base_w)      # the MTP layer is exported
    for layout in layouts:
        tp, ep, cp = layout[:3]
        pp = layout[3] if len(layout) > 3 else 1
        for losses, weights in run_ranks(_worker, 4, d, tp, ep, cp, False, pp, tied):
            for (a, _), (b, _) in zip(losses, base_losses):
                assert abs(a - b) < 3e-5, (layout, losses, base_losses)
            assert set(weights) == set(base_w)
            for k, v in base_w.items():
                assert torch.allclose(weights[k], v, rtol=0, atol=2e-6), (layout, k,
                                                                          (weights[k] - v).abs().max().item())


def test_mtp_tp2_ep2_and_cp2_match_single_process(tmp_path):
    _check(tmp_path, [(2, 2, 1), (1, 2, 2)])


def test_mtp_pp2_tp2_matches_single_process(tmp_path):
    """The last stage holds an embedding of its own for the MTP depths: a second copy of the first stage's matrix, which
    the checkpoint load has to fill (tensor-parallel shards: a random init would not match) and whose gradient is
    summed with the first stage's."""
    _check(tmp_path, [(2, 1, 1, 2)])


def test_mtp_tied_embeddings_pp2_tp2_matches_single_process(tmp_path):
    """Tied weights: on the last stage the MTP embedding and the head are one tensor, paired with the first stage's."""
    _check(tmp_path, [(2, 1, 1, 2)], tied=True)
