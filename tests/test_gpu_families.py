"""Hybrid / sparse-attention families on the GPU in bf16: the CUDA kernels they route through (causal conv1d, gated
RMSNorm, per-head norms, DSA indexer scores + top-k, attention, grouped GEMMs) against the same model in fp32 on the CPU
reference paths."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def _build(hf_cfg, dtype, device, seed=5, **kw):
    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    from mcore_bridge_b200.train.trainer import init_weights
    cfg = ModelConfig(**hf_to_mcore_config(hf_cfg), params_dtype=dtype, **kw)
    with torch.device(device):
        model = cfg.model_meta.loader(cfg).get_model_cls()(cfg)
    init_weights(model, 0.05, seed)
    return cfg, model


def _compare(hf_cfg, vocab, T=192, tol=6e-2, prep=None, **kw):
    _, ref = _build(hf_cfg, torch.float32, 'cpu', **kw)
    _, gpu = _build(hf_cfg, torch.bfloat16, 'cuda', **kw)
    if prep is not None:
        prep(ref)
    with torch.no_grad():       # identical weights: the bf16 model gets the rounded fp32 values
        for (n1, p1), (n2, p2) in zip(ref.named_parameters(), gpu.named_parameters()):
            assert n1 == n2
            p2.copy_(p1.to(torch.bfloat16))
            p1.copy_(p2.float().cpu())
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, vocab, (1, T), generator=g)
    labels = torch.randint(0, vocab, (1, T), generator=g)
    ref.train(), gpu.train()
    l_ref = ref(ids, labels=labels).mean()
    l_gpu = gpu(ids.to(DEV), labels=labels.to(DEV)).mean()
    l_ref.backward()
    l_gpu.backward()
    torch.cuda.synchronize()
    from mcore_bridge_b200.ops import _lib
    _lib.check_status()
    assert abs(l_ref.item() - l_gpu.item()) < 3e-2, (l_ref.item(), l_gpu.item())
    worst, bad = 0.0, []
    for (n, p1), (_, p2) in zip(ref.named_parameters(), gpu.named_parameters()):
        if p1.grad is None or p1.grad.abs().max() == 0:
            continue
        r = ((p2.grad.float().cpu() - p1.grad).norm() / p1.grad.norm()).item()
        worst = max(worst, r)
        # a router or indexer weight (and the scales in front of a router) feeds a discrete top-k: one selection that
        # flips under bf16 rounding moves its gradient by a whole token's contribution, so those only get a sanity bound
        discrete = any(k in n for k in ('router', 'indexer', 'experts_mlp.scale', 'per_expert_scale'))
        if r >= (0.75 if discrete else tol * 3):
            bad.append((n, round(r, 4)))
    assert not bad, bad
    return worst


def test_qwen3_next_hybrid_gpu_matches_cpu_reference():
    from transformers import Qwen3NextConfig
    c = Qwen3NextConfig(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                        intermediate_size=256, moe_intermediate_size=64, shared_expert_intermediate_size=64,
                        num_experts=8, num_experts_per_tok=2, linear_num_key_heads=2, linear_num_value_heads=4,
                        linear_key_head_dim=64, linear_value_head_dim=64, linear_conv_kernel_dim=4, vocab_size=256,
                        max_position_embeddings=512, full_attention_interval=4, partial_rotary_factor=0.25,
                        tie_word_embeddings=False, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
    _compare(c, 256)


def test_glm_dsa_gpu_matches_cpu_reference(monkeypatch):
    from transformers import GlmMoeDsaConfig
    c = GlmMoeDsaConfig(num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                        q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                        n_routed_experts=4, num_experts_per_tok=2, n_group=1, topk_group=1, moe_intermediate_size=32,
                        intermediate_size=128, mlp_layer_types=['dense', 'sparse'], n_shared_experts=1, vocab_size=256,
                        max_position_embeddings=512, index_n_heads=4, index_head_dim=128, index_topk=64,
                        tie_word_embeddings=False)
    # both the dense-masked and the gather-based sparse attention, each with the CUDA indexer + top-k for selection
    for min_t in ('100000', '0'):
        monkeypatch.setenv('MCB200_DSA_GATHER_MIN_T', min_t)
        _compare(c, 256, T=256, tol=8e-2)


def test_gemma4_gpu_matches_cpu_reference():
    """Sliding layers (windowed attention), global layers with their own head size on the tcgen05 attention kernel,
    shared-KV tail layers, the MoE branch on the grouped GEMMs and the per-layer input path."""
    from transformers import Gemma4TextConfig
    c = Gemma4TextConfig(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=6,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, global_head_dim=128,
                         num_global_key_value_heads=2, attention_k_eq_v=True,
                         layer_types=['sliding_attention', 'sliding_attention', 'full_attention'] * 2,
                         sliding_window=64, num_kv_shared_layers=2, use_double_wide_mlp=True,
                         hidden_size_per_layer_input=64, vocab_size_per_layer_input=256, enable_moe_block=True,
                         num_experts=4, top_k_experts=2, moe_intermediate_size=64, final_logit_softcapping=30.0,
                         max_position_embeddings=512, tie_word_embeddings=True, pad_token_id=0)

    def condition(model):
        with torch.no_grad():
            for layer in model.decoder.layers:
                # the router sees a unit-norm vector: with the generic small initialisation all four experts would
                # score within bf16 rounding of each other and the top-2 choice would be noise
                layer.experts_mlp.router.weight.mul_(60.0)
                # softmax scale is 1 and q / k are RMS-normalised: unit norm weights would give logits of the order
                # of sqrt(d) ~ 8-11, where bf16 rounding of q and k alone moves the probabilities by several percent
                attn = layer.self_attention
                attn.q_layernorm.weight.mul_(0.35)
                if attn.k_layernorm is not None:
                    attn.k_layernorm.weight.mul_(0.35)

    _compare(c, 256, T=256, tol=8e-2, prep=condition)


def _two_steps(name, seed, **kw):
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    cfg = model_config(name, None, params_dtype=torch.bfloat16, bf16=True, **kw)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=seed, clip_grad=1.0))
    ds = SyntheticPackedDataset(1024, 1024, seg_lo=96, seg_hi=512, seed=3, pin=False)
    losses = [float(tr.train_step([ds.next_microbatch() for _ in range(2)])) for _ in range(2)]
    torch.cuda.synchronize()
    weights = {n: p.detach().clone() for m in tr.models for n, p in m.named_parameters()}
    return losses, weights


@pytest.mark.parametrize('name,kw', [('qwen3_tiny', {}), ('qwen3_moe_tiny', {'moe_aux_loss_coeff': 1e-2})])
def test_training_steps_repeat_bit_for_bit(name, kw):
    """Two optimizer steps from the same seed and data, run twice in one process: losses and every weight must be
    identical bits.  A kernel whose result depends on the order in which CTAs or warps finish (atomics on floats, a
    race on a buffer) shows up here as a differing parameter."""
    l1, w1 = _two_steps(name, 11, **kw)
    l2, w2 = _two_steps(name, 11, **kw)
    assert l1 == l2, (l1, l2)
    bad = [n for n in w1 if not torch.equal(w1[n], w2[n])]
    assert not bad, bad[:8]
