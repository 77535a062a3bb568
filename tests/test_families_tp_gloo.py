"""TP=2 on gloo for the families whose attention normalises across heads (OLMoE: full-channel q/k norm with the
statistics reduced over TP) — logits and a sharded gradient equal the single-process model."""
import torch

from dist_utils import run_ranks


def _build():
    from transformers import OlmoeConfig, OlmoeForCausalLM
    torch.manual_seed(0)
    c = OlmoeConfig(vocab_size=512, hidden_size=128, intermediate_size=64, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=4, num_experts=8, num_experts_per_tok=2,
                    max_position_embeddings=256, pad_token_id=0, norm_topk_prob=False)
    hf = OlmoeForCausalLM(c).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            p.normal_(0, 0.02) if p.dim() >= 2 else p.normal_(1.0, 0.1)
    return c, hf


def _worker(rank, world, ckpt):
    from transformers import AutoConfig

    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    ps.initialize_model_parallel(tensor_model_parallel_size=2, expert_tensor_parallel_size=1)
    c = AutoConfig.from_pretrained(ckpt)
    cfg = ModelConfig(**hf_to_mcore_config(c), params_dtype=torch.float32, tensor_model_parallel_size=2,
                      expert_tensor_parallel_size=1, sequence_parallel=True)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], ckpt)
    ids = torch.randint(0, 512, (2, 64), generator=torch.Generator().manual_seed(1))
    labels = torch.randint(0, 512, (2, 64), generator=torch.Generator().manual_seed(2))
    loss = model(ids, labels=labels)
    loss.mean().backward()
    attn = model.decoder.layers[0].self_attention
    return loss.detach(), attn.q_norm.weight.grad.clone(), attn.k_norm.weight.grad.clone()


def test_olmoe_tp2_matches_transformers(tmp_path):
    c, hf = _build()
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    ids = torch.randint(0, 512, (2, 64), generator=torch.Generator().manual_seed(1))
    labels = torch.randint(0, 512, (2, 64), generator=torch.Generator().manual_seed(2))
    logits = hf(ids).logits
    ref = torch.nn.functional.cross_entropy(logits.view(-1, 512), labels.view(-1), reduction='none').view(2, 64)
    ref.mean().backward()
    res = run_ranks(_worker, 2, d)
    a = hf.model.layers[0].self_attn
    for r in range(2):
        assert torch.allclose(res[r][0], ref.detach(), atol=2e-5)
    # the norm weights are sharded by head: the two ranks' gradients concatenate to the full gradient
    assert torch.allclose(torch.cat([res[0][1], res[1][1]]), a.q_norm.weight.grad, atol=1e-6)
    assert torch.allclose(torch.cat([res[0][2], res[1][2]]), a.k_norm.weight.grad, atol=1e-6)
