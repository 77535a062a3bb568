"""Layout equivalence (see ``test_parallel_equivalence_gloo.py``) for the hybrid and the MLA / DSA-style families: two
optimizer steps on four gloo ranks against one process, weights through the checkpoint bridge."""
import torch

from dist_utils import run_ranks

STEPS, GLOBAL_MB = 2, 4
_BASE = {}      # single-process results per model (the checkpoint is seeded, so they do not depend on the test)


def _worker(rank, world, ckpt, tp, ep, pp, cp, over):
    from transformers import AutoConfig

    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=1, pipeline_model_parallel_size=pp,
                                 context_parallel_size=cp)
    kw = hf_to_mcore_config(AutoConfig.from_pretrained(ckpt))
    kw.update(over or {})
    cfg = ModelConfig(**kw, params_dtype=torch.float32, tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                      expert_tensor_parallel_size=1, pipeline_model_parallel_size=pp, context_parallel_size=cp,
                      sequence_parallel=tp > 1)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=1.0))
    cfg.bridge.load_weights(tr.models, ckpt)
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    dp, dp_rank = ps.get_world_size('dp'), ps.get_rank_in('dp') if ps.get_world_size('dp') > 1 else 0
    ds = SyntheticPackedDataset(256, 256, seg_lo=32, seg_hi=128, seed=3, pin=False, segment_multiple=4)
    losses = []
    for _ in range(STEPS):
        mbs = [ds.next_microbatch() for _ in range(GLOBAL_MB)]
        losses.append(tr.train_step(mbs[dp_rank::dp]))
    weights = {k: v.clone() for k, v in cfg.bridge.export_weights(tr.models)}
    return losses, weights, ps.is_pipeline_last_stage()


def _check(tmp_path, hf, tp=1, ep=1, pp=1, cp=1, over=None, atol=2e-6):
    torch.manual_seed(0)
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0 if 'norm' in n else 0.0, 0.05)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    key = (type(hf).__name__, hf.config.to_json_string(), repr(sorted((over or {}).items())))
    if key not in _BASE:
        _BASE[key] = run_ranks(_worker, 1, d, 1, 1, 1, 1, over)[0]
    base_losses, base_w, _ = _BASE[key]
    res = run_ranks(_worker, 4, d, tp, ep, pp, cp, over)
    for losses, weights, last_stage in res:
        if last_stage:
            for a, b in zip(losses, base_losses):
                assert abs(a - b) < 3e-5, (losses, base_losses)
        assert set(weights) == set(base_w)
        for k, v in base_w.items():
            assert torch.allclose(weights[k], v, rtol=0, atol=atol), (k, (weights[k] - v).abs().max().item())


def _qwen3_next(k_heads=2, v_heads=4):
    from transformers import Qwen3NextConfig, Qwen3NextForCausalLM
    c = Qwen3NextConfig(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                        intermediate_size=256, moe_intermediate_size=64, shared_expert_intermediate_size=64,
                        num_experts=8, num_experts_per_tok=2, linear_num_key_heads=k_heads, linear_num_value_heads=v_heads,
                        linear_key_head_dim=32, linear_value_head_dim=32, linear_conv_kernel_dim=4, vocab_size=256,
                        max_position_embeddings=512, full_attention_interval=4, partial_rotary_factor=0.25,
                        tie_word_embeddings=False, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
    return Qwen3NextForCausalLM(c).float()


def _deepseek_v3():
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    c = DeepseekV3Config(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                         q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                         n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1, moe_intermediate_size=32,
                         intermediate_size=128, first_k_dense_replace=1, n_shared_experts=1, vocab_size=256,
                         max_position_embeddings=512, tie_word_embeddings=False, routed_scaling_factor=1.5)
    return DeepseekV3ForCausalLM(c).float()


def test_qwen3_next_tp2_dp2_matches_single_process(tmp_path):
    _check(tmp_path, _qwen3_next(), tp=2, over={'moe_aux_loss_coeff': 1e-2})


def test_qwen3_next_cp2_ep2_matches_single_process(tmp_path):
    _check(tmp_path, _qwen3_next(), cp=2, ep=2, over={'moe_aux_loss_coeff': 1e-2})


def test_deepseek_v3_tp2_ep2_matches_single_process(tmp_path):
    _check(tmp_path, _deepseek_v3(), tp=2, ep=2, over={'moe_aux_loss_coeff': 1e-2})


def _gemma4():
    from transformers import Gemma4ForCausalLM, Gemma4TextConfig
    c = Gemma4TextConfig(vocab_size=256, hidden_size=64, intermediate_size=96, num_hidden_layers=6,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, global_head_dim=32,
                         num_global_key_value_heads=2, attention_k_eq_v=True,
                         layer_types=['sliding_attention', 'sliding_attention', 'full_attention'] * 2,
                         sliding_window=32, num_kv_shared_layers=2, use_double_wide_mlp=True,
                         hidden_size_per_layer_input=8, vocab_size_per_layer_input=256, enable_moe_block=True,
                         num_experts=4, top_k_experts=2, moe_intermediate_size=32, final_logit_softcapping=30.0,
                         max_position_embeddings=512, tie_word_embeddings=True, pad_token_id=0)
    return Gemma4ForCausalLM(c).float()


def test_gemma4_pp2_dp2_matches_single_process(tmp_path):
    """Per-layer inputs and the shared keys / values of the full-attention type cross the stage boundary (the sliding
    type's are produced on the second stage), gradients come back through the packed tensor."""
    _check(tmp_path, _gemma4(), pp=2)


def test_gemma4_tp2_pp2_matches_single_process(tmp_path):
    _check(tmp_path, _gemma4(), tp=2, pp=2)


def test_gemma4_tp2_dp2_matches_single_process(tmp_path):
    """The per-layer inputs are computed identically on both tensor-parallel ranks and consumed column by column: the
    gradients of the table, the projection and its norm need the other rank's columns too."""
    _check(tmp_path, _gemma4(), tp=2)


def _glm_dsa():
    from transformers import GlmMoeDsaConfig, GlmMoeDsaForCausalLM
    c = GlmMoeDsaConfig(num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                        q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                        n_routed_experts=4, num_experts_per_tok=2, n_group=1, topk_group=1, moe_intermediate_size=32,
                        intermediate_size=128, mlp_layer_types=['dense', 'sparse'], n_shared_experts=1, vocab_size=256,
                        max_position_embeddings=512, index_n_heads=4, index_head_dim=32, index_topk=16,
                        tie_word_embeddings=False)
    return GlmMoeDsaForCausalLM(c).float()


def test_glm_dsa_cp2_ep2_matches_single_process(tmp_path):
    """Sparse (top-16 keys) MLA attention with the queries of this rank's zig-zag chunks against the gathered keys of
    the whole stream, indexer keys included."""
    _check(tmp_path, _glm_dsa(), cp=2, ep=2)


def test_glm_dsa_tp2_ep2_matches_single_process(tmp_path):
    _check(tmp_path, _glm_dsa(), tp=2, ep=2)


def _gpt_oss():
    from transformers import GptOssConfig, GptOssForCausalLM
    c = GptOssConfig(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                     intermediate_size=64, num_local_experts=4, num_experts_per_tok=2, vocab_size=256,
                     max_position_embeddings=512, sliding_window=32, tie_word_embeddings=False,
                     layer_types=['sliding_attention', 'full_attention'] * 2, rope_parameters=None)
    return GptOssForCausalLM(c).float()


def test_gpt_oss_tp2_dp2_matches_single_process(tmp_path):
    """Learnable softmax sinks (sharded by head), sliding-window layers, biased expert projections."""
    _check(tmp_path, _gpt_oss(), tp=2)


def test_gpt_oss_cp2_ep2_matches_single_process(tmp_path):
    _check(tmp_path, _gpt_oss(), cp=2, ep=2)


def test_qwen3_next_tp2_cp2_matches_single_process(tmp_path):
    # the linear-attention heads are split over tp and, inside the layer, once more over cp
    _check(tmp_path, _qwen3_next(4, 8), tp=2, cp=2, over={'moe_aux_loss_coeff': 1e-2})


def test_glm_dsa_indexer_loss_tp2_ep2_matches_single_process(tmp_path):
    """Training the DSA indexer (KL towards the attention distribution): the target sums the heads of both
    tensor-parallel ranks, so every rank computes the same loss for the replicated indexer."""
    _check(tmp_path, _glm_dsa(), tp=2, ep=2, over={'dsa_indexer_loss_coeff': 0.1})
