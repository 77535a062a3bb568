"""Hyper-connections (n residual streams) and hash-routed MoE layers: invariants of the arithmetic, equivalence with
the single-stream model at the identity setting, gradients, and the checkpoint keys."""
import torch


def _cfg(**kw):
    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    from mcore_bridge_b200.train.presets import hf_config
    return ModelConfig(**{**hf_to_mcore_config(hf_config('qwen3_moe_tiny')), 'params_dtype': torch.float32, **kw})


def test_sinkhorn_gives_doubly_stochastic_maps():
    from mcore_bridge_b200.layers.hyper_connection import HyperConnection, sinkhorn
    torch.manual_seed(0)
    m = sinkhorn(torch.rand(5, 4, 4) + 0.05, 30)
    assert torch.allclose(m.sum(-1), torch.ones(5, 4), atol=1e-4) and torch.allclose(m.sum(-2), torch.ones(5, 4), atol=1e-4)
    cfg = _cfg(enable_hyper_connections=True, num_residual_streams=4)
    hc = HyperConnection(cfg)
    with torch.no_grad():
        hc.mapping_proj.weight.normal_(0, 0.05)
        hc.alpha_res.fill_(1.0)
        hc.bias.zero_()
    streams = torch.randn(7, 4 * cfg.hidden_size)
    x, post, res = hc.pre(streams)
    assert x.shape == (7, cfg.hidden_size) and post.shape == (7, 4) and res.shape == (7, 4, 4)
    assert torch.allclose(res.sum(-1), torch.ones(7, 4), atol=1e-2) and torch.allclose(res.sum(-2), torch.ones(7, 4), atol=1e-3)
    assert (res >= 0).all()


def test_identity_setting_reproduces_single_stream_model():
    """With the maps at their initial (identity) values every stream carries the ordinary residual, so the model's
    logits equal those of the same weights without hyper-connections."""
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.trainer import init_weights
    base_cfg = _cfg()
    base = get_mcore_model(base_cfg)[0]
    init_weights(base, 0.05, 1)
    hc_cfg = _cfg(enable_hyper_connections=True, num_residual_streams=4)
    model = get_mcore_model(hc_cfg)[0]
    missing, unexpected = model.load_state_dict(base.state_dict(), strict=False)
    assert not unexpected and all('hyper_connection' in k or 'hc_head' in k for k in missing)
    ids = torch.randint(0, 1024, (2, 48), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ref, out = base.eval()(ids), model.eval()(ids)
    assert (ref - out).abs().max().item() < 2e-3          # res is the identity up to exp(-8) off-diagonal mass
    # away from the identity setting the streams differ and every hyper-connection parameter gets a gradient
    with torch.no_grad():
        for n, p in model.named_parameters():
            if 'mapping_proj' in n:
                p.normal_(0, 0.05)
    model.train()(ids, labels=ids).mean().backward()
    for n, p in model.named_parameters():
        if 'hyper_connection' in n or 'hc_head' in n:
            assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, n


def test_hyper_connection_and_hash_table_checkpoint_keys(tmp_path):
    from safetensors.torch import load_file

    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.trainer import init_weights
    cfg = _cfg(enable_hyper_connections=True, num_residual_streams=4, moe_n_hash_layers=1)
    model = get_mcore_model(cfg)[0]
    init_weights(model, 0.05, 1)
    r0, r1 = model.decoder.layers[0].mlp.router, model.decoder.layers[1].mlp.router
    assert r0.is_hash_layer and not r1.is_hash_layer
    with torch.no_grad():
        r0.tid2eid.copy_(torch.randint(0, cfg.num_moe_experts, r0.tid2eid.shape, generator=torch.Generator().manual_seed(2)))
        for n, p in model.named_parameters():
            if 'hyper_connection' in n or 'hc_head' in n:
                p.normal_(0, 0.1)
    d = str(tmp_path / 'ckpt')
    cfg.bridge.save_weights([model], d)
    sd = load_file(f'{d}/model.safetensors')
    for key in ('model.layers.0.hc_attn_fn', 'model.layers.0.hc_attn_base', 'model.layers.0.hc_attn_scale',
                'model.layers.1.hc_ffn_fn', 'model.hc_head_fn', 'model.hc_head_scale', 'model.layers.0.mlp.gate.tid2eid'):
        assert key in sd, key
    assert sd['model.layers.0.hc_attn_scale'].shape == (3,) and sd['model.hc_head_scale'].shape == (1,)
    assert 'model.layers.1.mlp.gate.tid2eid' not in sd
    model2 = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model2], d)
    ids = torch.randint(0, 1024, (2, 40), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        assert torch.equal(model.eval()(ids), model2.eval()(ids))


def test_hash_routing_uses_the_table():
    from mcore_bridge_b200.layers.moe import TopKRouter
    cfg = _cfg(moe_n_hash_layers=1)
    r = TopKRouter(cfg, is_hash_layer=True)
    with torch.no_grad():
        r.weight.normal_(0, 0.1)
        r.tid2eid.copy_(torch.stack([torch.arange(cfg.padded_vocab_size) % 8, (torch.arange(cfg.padded_vocab_size) + 3) % 8], 1))
    ids = torch.tensor([[5, 9, 1023, 0]])
    x = torch.randn(4, cfg.hidden_size)
    probs, idx = r(x, input_ids=ids)
    assert torch.equal(idx, r.tid2eid[ids.reshape(-1)])
    scores = torch.softmax(r.gating(x).float(), -1)
    assert torch.allclose(probs.float(), scores.gather(1, idx), atol=1e-6)


def test_cpu_offloading_gives_the_same_gradients():
    """``cpu_offloading`` only moves where saved activations live."""
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.trainer import init_weights
    grads = []
    ids = torch.randint(0, 1024, (2, 48), generator=torch.Generator().manual_seed(0))
    for off in (False, True):
        cfg = _cfg(cpu_offloading=off, cpu_offloading_num_layers=1)
        model = get_mcore_model(cfg)[0].train()
        init_weights(model, 0.05, 1)
        model(ids, labels=ids).mean().backward()
        grads.append({n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None})
    assert grads[0].keys() == grads[1].keys()
    for n in grads[0]:
        assert torch.equal(grads[0][n], grads[1][n]), n


def test_fine_grained_offloading_moves_saved_tensors_and_keeps_gradients():
    """``offload_modules`` names sub-blocks whose saved tensors live on the host between forward and backward: the
    pack hook runs only while a named sub-block runs, and gradients do not change."""
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.trainer import init_weights
    ids = torch.randint(0, 1024, (2, 48), generator=torch.Generator().manual_seed(0))
    grads, packed = [], []
    for mods in (None, ['mlp_norm', 'moe_act'], ['core_attn']):
        cfg = _cfg(fine_grained_activation_offloading=mods is not None, offload_modules=mods)
        model = get_mcore_model(cfg)[0].train()
        init_weights(model, 0.05, 1)
        seen = []
        orig = torch.autograd.graph.save_on_cpu

        class Spy(orig):
            def __init__(self, *a, **k):
                seen.append(1)
                super().__init__(*a, **k)
        torch.autograd.graph.save_on_cpu = Spy
        try:
            model(ids, labels=ids).mean().backward()
        finally:
            torch.autograd.graph.save_on_cpu = orig
        packed.append(len(seen))
        grads.append({n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None})
    n_layers = _cfg().num_layers
    assert packed == [0, n_layers, n_layers]          # one sub-block per layer each time
    for g in grads[1:]:
        assert g.keys() == grads[0].keys()
        for n in g:
            assert torch.equal(g[n], grads[0][n]), n


def test_unbuilt_options_are_refused():
    import pytest
    with pytest.raises(NotImplementedError, match='compressed attention layers'):
        _cfg(csa_compress_ratios=[0, 4])
    with pytest.raises(NotImplementedError, match='multi-token-prediction'):
        _cfg(experimental_attention_variant='dsv4_hybrid', mtp_num_layers=1)
