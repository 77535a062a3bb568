"""Gemma-4 text decoder against ``transformers.Gemma4ForCausalLM``: logits, loss and gradients of a model that uses
every optional piece (two layer types with different head sizes, k = v global attention, shared-KV tail layers with
the double-wide MLP, the MoE branch, per-layer inputs, layer scalars, soft-capped logits), the plain variant, the
checkpoint round trip, and TP = 2 (+ sequence parallel) on gloo."""
import pytest
import torch

from dist_utils import run_ranks

LAYER_TYPES = ['sliding_attention', 'sliding_attention', 'full_attention'] * 2


def _hf(full: bool, seed: int = 0):
    from transformers import Gemma4ForCausalLM, Gemma4TextConfig
    torch.manual_seed(seed)
    extra = dict(num_global_key_value_heads=2, attention_k_eq_v=True, num_kv_shared_layers=2, use_double_wide_mlp=True,
                 hidden_size_per_layer_input=8, vocab_size_per_layer_input=128, enable_moe_block=True, num_experts=4,
                 top_k_experts=2, moe_intermediate_size=32, final_logit_softcapping=30.0) if full else \
        dict(hidden_size_per_layer_input=0)
    c = Gemma4TextConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=6,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, global_head_dim=32,
                         layer_types=list(LAYER_TYPES), sliding_window=8, max_position_embeddings=128,
                         tie_word_embeddings=True, pad_token_id=0, **extra)
    hf = Gemma4ForCausalLM(c).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
            else:
                p.mul_(3.0)
        for n, b in hf.named_buffers():
            if n.endswith('layer_scalar'):
                b.fill_(0.9)
    return c, hf


def _ours(ckpt, **kw):
    from transformers import AutoConfig

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    cfg = ModelConfig(**hf_to_mcore_config(AutoConfig.from_pretrained(ckpt)), params_dtype=torch.float32, **kw)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], ckpt)
    return cfg, model


def _close(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item() < 1e-4


def _batch():
    g = torch.Generator().manual_seed(1)
    return torch.randint(1, 128, (2, 24), generator=g), torch.randint(1, 128, (2, 24), generator=g)


def _hf_loss(hf, ids, labels):
    logits = hf(ids, use_cache=True).logits
    return logits, torch.nn.functional.cross_entropy(logits.view(-1, 128), labels.view(-1), reduction='none').view(2, -1)


@pytest.mark.parametrize('full', [True, False])
def test_gemma4_matches_transformers(tmp_path, full):
    c, hf = _hf(full)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    cfg, model = _ours(d)
    ids, labels = _batch()
    ref_logits, ref_loss = _hf_loss(hf, ids, labels)
    ref_loss.mean().backward()
    logits = model(ids, runtime_gather_output=True)
    assert torch.allclose(logits, ref_logits, atol=5e-5), (logits - ref_logits).abs().max()
    loss = model(ids, labels=labels)
    assert torch.allclose(loss, ref_loss.detach(), atol=5e-5)
    loss.mean().backward()
    # a gradient from each special path
    l0, h0 = model.decoder.layers[0], hf.model.layers[0]
    assert _close(l0.self_attention.q_layernorm.weight.grad, h0.self_attn.q_norm.weight.grad)
    assert _close(l0.post_feedforward_layernorm.weight.grad, h0.post_feedforward_layernorm.weight.grad)
    assert _close(model.embedding.word_embeddings.weight.grad, hf.model.embed_tokens.weight.grad)
    if full:
        assert _close(l0.experts_mlp.scale.grad, h0.router.scale.grad)
        assert _close(l0.experts_mlp.per_expert_scale.grad, h0.router.per_expert_scale.grad)
        assert _close(l0.per_layer_projection.weight.grad, h0.per_layer_projection.weight.grad)
        assert _close(model.embed_tokens_per_layer.weight.grad, hf.model.embed_tokens_per_layer.weight.grad)
        l5, h5 = model.decoder.layers[5], hf.model.layers[5]          # shared-KV layer: queries only, wide MLP
        assert l5.self_attention.is_kv_shared and l5.self_attention.k_layernorm is None
        assert _close(l5.self_attention.linear_qkv.weight.grad, h5.self_attn.q_proj.weight.grad)
        assert l5.mlp.linear_fc2.weight.shape[1] == 2 * 96


def test_gemma4_checkpoint_round_trip(tmp_path):
    c, hf = _hf(True)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    cfg, model = _ours(d)
    out = dict(cfg.bridge.export_weights([model]))
    sd = hf.state_dict()
    # the tail layers attend to an earlier layer's keys and values: their own k / v projections are not part of
    # the model (nor of the export); the tied head is stored once
    skipped = {k for k in sd if any(f'layers.{i}.self_attn.{n}' in k for i in (4, 5)
                                    for n in ('k_proj', 'v_proj', 'k_norm'))} | {'lm_head.weight'}
    assert set(out) == set(sd) - skipped, (set(out) ^ (set(sd) - skipped))
    for k, v in out.items():
        assert torch.equal(v, sd[k]), k


def _tp_worker(rank, world, ckpt, sp):
    from mcore_bridge_b200.parallel import state as ps
    ps.initialize_model_parallel(tensor_model_parallel_size=2, expert_tensor_parallel_size=1)
    cfg, model = _ours(ckpt, tensor_model_parallel_size=2, expert_tensor_parallel_size=1, sequence_parallel=sp)
    ids, labels = _batch()
    loss = model(ids, labels=labels)
    loss.mean().backward()
    l0 = model.decoder.layers[0]
    return (loss.detach(), l0.self_attention.q_layernorm.weight.grad.clone(), l0.experts_mlp.scale.grad.clone(),
            l0.per_layer_projection.weight.grad.clone())


@pytest.mark.parametrize('sp', [False, True])
def test_gemma4_tp2_matches_transformers(tmp_path, sp):
    c, hf = _hf(True)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    ids, labels = _batch()
    _, ref_loss = _hf_loss(hf, ids, labels)
    ref_loss.mean().backward()
    res = run_ranks(_tp_worker, 2, d, sp)
    h0 = hf.model.layers[0]
    for r in range(2):
        assert torch.allclose(res[r][0], ref_loss.detach(), atol=5e-5)
    # replicated weights hold partial gradients that the optimizer sums over the TP group
    assert _close(res[0][1] + res[1][1], h0.self_attn.q_norm.weight.grad)
    # the MoE branch sees every token on both ranks without sequence parallelism, a token shard with it
    assert _close(res[0][2] + res[1][2] if sp else res[0][2], h0.router.scale.grad)
    # a row-parallel weight is split on its input dimension
    assert _close(torch.cat([res[0][3], res[1][3]], dim=1), h0.per_layer_projection.weight.grad)


def test_gemma4_multimodal_matches_transformers(tmp_path):
    """Image soft tokens written into the scaled text embeddings; the per-layer inputs come from the ids with the
    placeholders replaced by the padding id and from the merged embeddings."""
    from transformers import AutoConfig, Gemma4Config, Gemma4ForConditionalGeneration

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    torch.manual_seed(0)
    text = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, global_head_dim=32,
                layer_types=['sliding_attention', 'sliding_attention', 'full_attention'], sliding_window=8,
                hidden_size_per_layer_input=8, vocab_size_per_layer_input=128, max_position_embeddings=128,
                pad_token_id=0)
    vision = dict(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                  num_key_value_heads=2, head_dim=16, pooling_kernel_size=2, patch_size=4, position_embedding_size=16)
    c = Gemma4Config(text_config=text, vision_config=vision, audio_config=None, image_token_id=120,
                     video_token_id=121, audio_token_id=122, tie_word_embeddings=True)
    hf = Gemma4ForConditionalGeneration(c).float().eval()
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    pv = torch.randn(1, 16, 3 * 4 * 4)
    pos = torch.stack(torch.meshgrid(torch.arange(4), torch.arange(4), indexing='xy'), -1).reshape(1, 16, 2)
    ids = torch.randint(1, 100, (1, 20))
    ids[0, 3:7] = 120
    with torch.no_grad():
        ref = hf(input_ids=ids, pixel_values=pv, image_position_ids=pos, use_cache=True).logits
    cfg = ModelConfig(**hf_to_mcore_config(AutoConfig.from_pretrained(d)), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], d)
    model.eval()
    with torch.no_grad():
        out = model(ids, pixel_values=pv, image_position_ids=pos, runtime_gather_output=True)
    assert torch.allclose(out, ref, atol=5e-5), (out - ref).abs().max()
    exported = dict(cfg.bridge.export_weights([model]))
    sd = hf.state_dict()
    assert set(exported) == set(sd) - {'lm_head.weight'}, set(exported) ^ set(sd)
    for k, v in exported.items():
        assert torch.equal(v, sd[k]), k


def _tp4_worker(rank, world, ckpt):
    from mcore_bridge_b200.parallel import state as ps
    ps.initialize_model_parallel(tensor_model_parallel_size=4, expert_tensor_parallel_size=1)
    cfg, model = _ours(ckpt, tensor_model_parallel_size=4, expert_tensor_parallel_size=1, sequence_parallel=True)
    ids, labels = _batch()
    loss = model(ids, labels=labels)
    loss.mean().backward()
    a2 = model.decoder.layers[2].self_attention           # global layer: one KV head shared by all four ranks
    assert a2.kv_rep == 4 and model.decoder.layers[0].self_attention.kv_rep == 2
    return loss.detach(), a2.k_layernorm.weight.grad.clone(), a2.linear_qkv.weight.grad.clone()


def test_gemma4_tp4_more_ranks_than_kv_heads(tmp_path):
    from transformers import Gemma4ForCausalLM
    c, _ = _hf(True)
    c.num_global_key_value_heads = 1
    torch.manual_seed(3)
    hf = Gemma4ForCausalLM(c).float().eval()
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    ids, labels = _batch()
    _, ref_loss = _hf_loss(hf, ids, labels)
    ref_loss.mean().backward()
    res = run_ranks(_tp4_worker, 4, d)
    for r in range(4):
        assert torch.allclose(res[r][0], ref_loss.detach(), atol=5e-5)
    a = hf.model.layers[2].self_attn
    assert _close(sum(res[r][1] for r in range(4)), a.k_norm.weight.grad)
    # rows of the packed projection are [4 query heads | k] of the single group, split evenly over the ranks
    full = torch.cat([res[r][2] for r in range(4)], dim=0)
    assert _close(full, torch.cat([a.q_proj.weight.grad, a.k_proj.weight.grad], dim=0))
