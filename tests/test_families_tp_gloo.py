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


def _moe_worker(rank, world, ckpt, sp):
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.presets import hf_config
    ps.initialize_model_parallel(tensor_model_parallel_size=2)            # expert tensor parallel = 2 as well
    cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_moe_tiny')), params_dtype=torch.float32,
                      tensor_model_parallel_size=2, sequence_parallel=sp)
    assert ps.get_world_size('etp') == 2
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], ckpt)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1024, (2, 64), generator=g)
    labels = torch.randint(0, 1024, (2, 64), generator=g)
    loss = model(ids, labels=labels)
    loss.mean().backward()
    mlp = model.decoder.layers[0].mlp
    exported = {k: v.clone() for k, v in cfg.bridge.export_weights([model])}
    return (loss.detach(), mlp.experts.linear_fc2.weight.grad.clone(), mlp.router.weight.grad.clone(), exported)


def _check_moe_etp(tmp_path, sp):
    import os

    from safetensors.torch import load_file
    from transformers import Qwen3MoeForCausalLM

    from mcore_bridge_b200.train.presets import hf_config
    torch.manual_seed(0)
    c = hf_config('qwen3_moe_tiny')
    hf = Qwen3MoeForCausalLM(c).float()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.02) if p.dim() >= 2 else p.normal_(1.0, 0.1)
    d = str(tmp_path / 'ckpt')
    hf.save_pretrained(d)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1024, (2, 64), generator=g)
    labels = torch.randint(0, 1024, (2, 64), generator=g)
    logits = hf(ids).logits
    ref = torch.nn.functional.cross_entropy(logits.view(-1, 1024), labels.view(-1), reduction='none').view(2, 64)
    ref.mean().backward()
    res = run_ranks(_moe_worker, 2, d, sp)
    disk = load_file(os.path.join(d, 'model.safetensors'))
    for r in range(2):
        assert torch.allclose(res[r][0], ref.detach(), atol=2e-5)
        assert sorted(res[r][3]) == sorted(disk) and all(torch.equal(res[r][3][k], disk[k]) for k in disk)
    # fc2 of the experts is row-parallel over the expert-TP group: the shards' gradients concatenate on the input dim
    gate = hf.model.layers[0].mlp.gate.weight.grad
    got = res[0][2] + res[1][2] if sp else res[0][2]       # router sees local tokens under sequence parallelism
    assert torch.allclose(got, gate, atol=1e-6)
    fc2 = torch.cat([res[0][1], res[1][1]], dim=2)          # [E, H, F]
    experts = hf.model.layers[0].mlp.experts
    if hasattr(experts, 'down_proj'):
        want = experts.down_proj.grad
    else:
        want = torch.stack([e.down_proj.weight.grad for e in experts])
    assert torch.allclose(fc2, want, atol=1e-6)


def test_moe_expert_tensor_parallel_sp(tmp_path):
    _check_moe_etp(tmp_path, True)


def test_moe_expert_tensor_parallel_no_sp(tmp_path):
    _check_moe_etp(tmp_path, False)
