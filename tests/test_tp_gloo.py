"""TP=2 (+sequence parallel) on two gloo ranks equals the single-process model; export gathers shards."""
import torch

from dist_utils import run_ranks


def _worker(rank, world, ckpt_dir, sp, tp=2):
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.presets import hf_config
    ps.initialize_model_parallel(tensor_model_parallel_size=tp)
    cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_tiny')), params_dtype=torch.float32,
                      tensor_model_parallel_size=tp, sequence_parallel=sp)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], ckpt_dir)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1024, (2, 128), generator=g)
    labels = torch.randint(0, 1024, (2, 128), generator=g)
    loss = model(ids, labels=labels)
    loss.mean().backward()
    logits = model(ids, runtime_gather_output=True).detach()
    exported = {k: v.clone() for k, v in cfg.bridge.export_weights([model])}
    gq = model.decoder.layers[0].self_attention.linear_qkv.weight.grad.clone()
    gn = model.decoder.layers[0].self_attention.linear_qkv.layer_norm_weight.grad.clone()
    gqn = model.decoder.layers[0].self_attention.q_layernorm.weight.grad.clone()
    return loss.detach(), logits, exported, gq, gn, gqn


def _setup(tmp):
    from transformers import Qwen3ForCausalLM

    from mcore_bridge_b200.train.presets import hf_config
    torch.manual_seed(0)
    hf = Qwen3ForCausalLM(hf_config('qwen3_tiny')).float()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.02) if p.dim() >= 2 else p.normal_(1.0, 0.1)
    hf.save_pretrained(tmp)
    return hf


def _check(tmp_path, sp):
    import torch.distributed as dist
    d = str(tmp_path / 'ckpt')
    hf = _setup(d)
    res = run_ranks(_worker, 2, d, sp)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1024, (2, 128), generator=g)
    labels = torch.randint(0, 1024, (2, 128), generator=g)
    ref_logits = hf(ids).logits
    ref_loss = torch.nn.functional.cross_entropy(ref_logits.view(-1, 1024), labels.view(-1), reduction='none').view(2, 128)
    ref_loss.mean().backward()
    for r in range(2):
        loss, logits, exported, gq, gn, _ = res[r]
        assert torch.allclose(loss, ref_loss.detach(), atol=1e-5)
        assert torch.allclose(logits, ref_logits.detach(), atol=1e-5)
        sd = hf.state_dict()
        for k, v in exported.items():
            assert torch.equal(v, sd[k]), k
    # gradient of the TP-sharded qkv weight: rank shards concatenate to the interleaved full gradient
    from mcore_bridge_b200.bridge.gpt_bridge import qkv_to_mcore
    a = hf.model.layers[0].self_attn
    full = qkv_to_mcore(a.q_proj.weight.grad, a.k_proj.weight.grad, a.v_proj.weight.grad, 2)
    got = torch.cat([res[0][3], res[1][3]], dim=0)
    assert torch.allclose(got, full, atol=1e-6)
    # per-head q norm: replicated weight, each rank covers its own heads, the partial gradients sum to the full one
    assert torch.allclose(res[0][5] + res[1][5], hf.model.layers[0].self_attn.q_norm.weight.grad, atol=1e-6)
    # replicated norm weight: with SP each rank has a partial gradient that sums to the full one
    gn_ref = hf.model.layers[0].input_layernorm.weight.grad
    if sp:
        assert torch.allclose(res[0][4] + res[1][4], gn_ref, atol=1e-6)
    else:
        assert torch.allclose(res[0][4], gn_ref, atol=1e-6)


def test_tp2(tmp_path):
    _check(tmp_path, sp=False)


def test_tp2_sequence_parallel(tmp_path):
    _check(tmp_path, sp=True)


def test_tp4_more_ranks_than_kv_heads(tmp_path):
    """4 query heads / 2 KV heads on TP=4: two ranks share each KV head (the projection output is gathered on the
    last dim and re-sliced); loss, logits, export and the packed QKV weight gradient equal the dense model."""
    d = str(tmp_path / 'ckpt')
    hf = _setup(d)
    res = run_ranks(_worker, 4, d, True, 4)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1024, (2, 128), generator=g)
    labels = torch.randint(0, 1024, (2, 128), generator=g)
    ref_logits = hf(ids).logits
    ref_loss = torch.nn.functional.cross_entropy(ref_logits.view(-1, 1024), labels.view(-1), reduction='none').view(2, 128)
    ref_loss.mean().backward()
    sd = hf.state_dict()
    for r in range(4):
        loss, logits, exported, gq, gn, gqn = res[r]
        assert torch.allclose(loss, ref_loss.detach(), atol=1e-5)
        assert torch.allclose(logits, ref_logits.detach(), atol=1e-5)
        for k, v in exported.items():
            assert torch.equal(v, sd[k]), k
    from mcore_bridge_b200.bridge.gpt_bridge import qkv_to_mcore
    a = hf.model.layers[0].self_attn
    full = qkv_to_mcore(a.q_proj.weight.grad, a.k_proj.weight.grad, a.v_proj.weight.grad, 2)
    got = torch.cat([res[r][3] for r in range(4)], dim=0)
    assert torch.allclose(got, full, atol=1e-6)
    assert torch.allclose(sum(res[r][5] for r in range(4)), a.q_norm.weight.grad, atol=1e-6)
