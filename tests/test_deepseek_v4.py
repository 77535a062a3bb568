"""DeepSeek-V4 family (sliding-window layers): config parsing, the attention block against a plain restatement written
from the checkpoint's own tensors, the on-disk key layout with fp4 / fp8 expert weights, and the refusal of compressed
layers."""
import math

import pytest
import torch


class _HFConfig:
    """Stand-in for the checkpoint's ``config.json`` (the installed Transformers has no class for this family and its
    base class rejects the family's layer-type names)."""

    def __init__(self, **kw):
        self.__dict__.update(kw)

    def to_dict(self):
        return dict(self.__dict__)


def _hf_config(layer_types=('sliding_attention', 'sliding_attention'), **kw):
    fields = dict(
        model_type='deepseek_v4', vocab_size=512, hidden_size=64, num_hidden_layers=len(layer_types),
        num_attention_heads=4, head_dim=32, qk_rope_head_dim=8, q_lora_rank=24, o_groups=2, o_lora_rank=16,
        rms_norm_eps=1e-6, rope_theta=10000, max_position_embeddings=256, n_routed_experts=4, num_experts_per_tok=2,
        moe_intermediate_size=32, n_shared_experts=1, scoring_func='sigmoid', norm_topk_prob=True, hidden_act='silu',
        layer_types=list(layer_types), sliding_window=8, hc_mult=2, hc_sinkhorn_iters=4,
        compress_rates={'compressed_sparse_attention': 4, 'heavily_compressed_attention': 128},
        mlp_layer_types=['hash_moe'] + ['moe'] * (len(layer_types) - 1), tie_word_embeddings=False,
        rope_scaling={'main': None, 'compress': {'rope_type': 'yarn', 'factor': 4.0,
                                                 'original_max_position_embeddings': 64}})
    fields.update(kw)
    return _HFConfig(**fields)


def _model(**kw):
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.train.trainer import init_weights
    cfg = ModelConfig(**{**hf_to_mcore_config(_hf_config()), 'params_dtype': torch.float32, **kw})
    model = get_mcore_model(cfg)[0]
    init_weights(model, 0.05, 3)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith('attn_sink'):
                p.normal_(0, 0.5)
            if 'hyper_connection' in n or 'hc_head' in n:
                p.normal_(0, 0.1)
        for layer in model.decoder.layers:
            r = layer.mlp.router
            if r.is_hash_layer:
                r.tid2eid.copy_(torch.randint(0, cfg.num_moe_experts, r.tid2eid.shape,
                                              generator=torch.Generator().manual_seed(5)))
    return cfg, model


def test_config_and_layer_structure():
    from mcore_bridge_b200.layers.dsv4_attention import DSv4SelfAttention
    cfg, model = _model()
    assert cfg.experimental_attention_variant == 'dsv4_hybrid' and cfg.enable_hyper_connections
    assert cfg.csa_compress_ratios == [0, 0] and cfg.csa_window_size == 8 and cfg.moe_n_hash_layers == 1
    assert cfg.num_residual_streams == 2 and cfg.o_groups == 2 and cfg.o_lora_rank == 16
    attn = model.decoder.layers[0].self_attention
    assert isinstance(attn, DSv4SelfAttention)
    assert attn.linear_kv_proj.weight.shape == (32, 64) and attn.linear_o_group_proj.shape == (2 * 16, 4 * 32 // 2)
    assert attn.linear_proj.weight.shape == (64, 32) and attn.core_attention.attn_sink.shape == (4,)
    assert model.decoder.layers[0].mlp.router.is_hash_layer and not model.decoder.layers[1].mlp.router.is_hash_layer


def test_compressed_layers_are_refused():
    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    kw = hf_to_mcore_config(_hf_config(('sliding_attention', 'compressed_sparse_attention')))
    with pytest.raises(NotImplementedError, match='compressed attention'):
        ModelConfig(**kw)


def _attention_restated(x, w, window, eps=1e-6):
    """One sequence ``x [T, H]`` through the attention block, written directly from the checkpoint tensors ``w``
    (disk names), with the rotation done on complex pairs."""
    T = x.shape[0]
    nh, d, rot = 4, 32, 8

    def rms(t, weight=None):
        t = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)
        return t if weight is None else t * weight

    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot))
    ang = torch.arange(T).float()[:, None] * inv[None, :]
    rotor = torch.polar(torch.ones_like(ang), ang)                       # [T, rot/2]

    def rotate(t, conj=False):                                            # t [T, heads, d]
        tail = torch.view_as_complex(t[..., -rot:].reshape(T, -1, rot // 2, 2).contiguous())
        tail = tail * (rotor.conj() if conj else rotor)[:, None, :]
        return torch.cat([t[..., :-rot], torch.view_as_real(tail).reshape(T, -1, rot)], dim=-1)

    q = rms(x @ w['wq_a.weight'].T, w['q_norm.weight']) @ w['wq_b.weight'].T
    q = rotate(rms(q.view(T, nh, d)))
    kv = rotate(rms(x @ w['wkv.weight'].T, w['kv_norm.weight']).view(T, 1, d))[:, 0]
    s = torch.einsum('thd,sd->hts', q, kv) / math.sqrt(d)
    pos = torch.arange(T)
    allowed = (pos[None, :] <= pos[:, None]) & (pos[:, None] - pos[None, :] < window)
    s = s.masked_fill(~allowed[None], float('-inf'))
    s = torch.cat([s, w['attn_sink'].view(nh, 1, 1).expand(nh, T, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)[..., :-1]
    o = rotate(torch.einsum('hts,sd->thd', p, kv), conj=True)
    g, r = 2, 16
    wo_a = w['wo_a.weight'].view(g, r, -1)
    y = torch.einsum('tgd,grd->tgr', o.reshape(T, g, -1), wo_a).reshape(T, g * r)
    return y @ w['wo_b.weight'].T


def test_attention_block_matches_restatement_and_disk_layout(tmp_path):
    from safetensors.torch import load_file

    from mcore_bridge_b200.layers.context import ForwardContext
    cfg, model = _model()
    d = str(tmp_path / 'ckpt')
    cfg.bridge.save_weights([model], d)
    sd = load_file(f'{d}/model.safetensors')
    # disk layout: no 'model.' prefix, family-specific names
    for key in ('embed.weight', 'head.weight', 'norm.weight', 'hc_head_fn', 'layers.0.attn_norm.weight',
                'layers.0.ffn_norm.weight', 'layers.0.attn.wq_a.weight', 'layers.0.attn.q_norm.weight',
                'layers.0.attn.wq_b.weight', 'layers.0.attn.wkv.weight', 'layers.0.attn.kv_norm.weight',
                'layers.0.attn.attn_sink', 'layers.0.attn.wo_a.weight', 'layers.0.attn.wo_b.weight',
                'layers.0.hc_attn_fn', 'layers.0.hc_ffn_scale', 'layers.0.ffn.gate.weight', 'layers.0.ffn.gate.tid2eid',
                'layers.0.ffn.experts.0.w1.weight', 'layers.0.ffn.experts.3.w2.weight',
                'layers.0.ffn.shared_experts.w3.weight', 'layers.1.ffn.gate.bias'):
        assert key in sd, key
    assert 'layers.0.ffn.gate.bias' not in sd and 'layers.1.ffn.gate.tid2eid' not in sd
    assert not any(k.startswith('model.') for k in sd)
    # the attention block against the restatement, on two packed sequences
    attn = model.decoder.layers[1].self_attention
    w = {k[len('layers.1.attn.'):]: v for k, v in sd.items() if k.startswith('layers.1.attn.')}
    torch.manual_seed(0)
    lens = [19, 13]
    x = torch.randn(sum(lens), cfg.hidden_size)
    pos = torch.cat([torch.arange(n) for n in lens])
    cos, sin = model.rotary_pos_emb(pos)
    ctx = ForwardContext(cu_seqlens=torch.tensor([0, 19, 32], dtype=torch.int32), max_seqlen=19, cos=cos, sin=sin,
                         position_ids=pos)
    with torch.no_grad():
        got = attn(x, ctx)
        want = torch.cat([_attention_restated(x[:19], w, 8), _attention_restated(x[19:], w, 8)])
    assert (got - want).abs().max().item() < 2e-5
    # the window matters at these lengths and the sink changes the result
    with torch.no_grad():
        assert (torch.cat([_attention_restated(x[:19], w, 64), _attention_restated(x[19:], w, 64)]) - want
                ).abs().max().item() > 1e-4
    # load back: same logits; gradients reach every attention parameter
    cfg2, model2 = _model()
    with torch.no_grad():
        for p in model2.parameters():
            p.add_(0.3)
    cfg2.bridge.load_weights([model2], d)
    ids = torch.randint(0, 512, (2, 24), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        a, b = model.eval()(ids), model2.eval()(ids)
    assert torch.equal(a, b)
    model.train()(ids, labels=ids).mean().backward()
    for n, p in model.decoder.layers[0].self_attention.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, n


def test_fp4_and_fp8_expert_weights_are_dequantised_on_load(tmp_path):
    from safetensors.torch import load_file, save_file

    from mcore_bridge_b200.utils.dequantizer import _FP4_VALUES
    cfg, model = _model()
    d = str(tmp_path / 'ckpt')
    cfg.bridge.save_weights([model], d)
    sd = load_file(f'{d}/model.safetensors')
    lut = torch.tensor(_FP4_VALUES[:8])
    expect = {}
    for key in [k for k in sd if '.experts.' in k and k.startswith('layers.0.')]:
        wt = sd.pop(key).float()                                  # [rows, cols], cols a multiple of 32
        blocks = wt.reshape(wt.shape[0], -1, 32)
        exp = torch.ceil(torch.log2(blocks.abs().amax(-1, keepdim=True).clamp(min=2.0**-100) / 6.0))
        scaled = blocks / torch.exp2(exp)
        code = (scaled.abs().unsqueeze(-1) - lut).abs().argmin(-1) + (scaled < 0).long() * 8
        code = code.reshape(wt.shape[0], -1).to(torch.uint8)
        sd[key] = (code[:, 0::2] | (code[:, 1::2] << 4)).view(torch.int8).contiguous()
        sd[key[:-len('.weight')] + '.scale'] = torch.exp2(exp).squeeze(-1).contiguous()
        vals = torch.tensor(_FP4_VALUES)[code.long()].reshape(wt.shape[0], -1, 32) * torch.exp2(exp)
        expect[key] = vals.reshape(wt.shape)
    for key in [k for k in sd if '.experts.' in k and k.startswith('layers.1.') and k.endswith('.weight')]:
        wt = sd.pop(key).float()
        scale = wt.abs().amax().clamp(min=1e-8) / 448.0
        q = (wt / scale).to(torch.float8_e4m3fn)
        sd[key] = q
        sd[key[:-len('.weight')] + '.scale'] = scale.reshape(1, 1)
        expect[key] = q.float() * scale
    save_file(sd, f'{d}/model.safetensors')
    cfg2, model2 = _model()
    cfg2.bridge.load_weights([model2], d)
    ex = model2.decoder.layers[0].mlp.experts
    w1 = torch.cat([expect['layers.0.ffn.experts.2.w1.weight'], expect['layers.0.ffn.experts.2.w3.weight']])
    assert torch.allclose(ex.linear_fc1.weight[2], w1, atol=1e-6)
    assert torch.allclose(ex.linear_fc2.weight[1], expect['layers.0.ffn.experts.1.w2.weight'], atol=1e-6)
    ex1 = model2.decoder.layers[1].mlp.experts
    assert torch.allclose(ex1.linear_fc2.weight[3], expect['layers.1.ffn.experts.3.w2.weight'], atol=1e-6)


# ------------------------------------------------------------------ parallel layouts against one process (gloo)
def _train_worker(rank, world, ckpt, tp, ep, cp, pp=1):
    from mcore_bridge_b200 import ModelConfig, hf_to_mcore_config
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=1, context_parallel_size=cp,
                                 pipeline_model_parallel_size=pp)
    cfg = ModelConfig(**hf_to_mcore_config(_hf_config()), params_dtype=torch.float32, tensor_model_parallel_size=tp,
                      expert_model_parallel_size=ep, expert_tensor_parallel_size=1, context_parallel_size=cp,
                      pipeline_model_parallel_size=pp, sequence_parallel=tp > 1, moe_aux_loss_coeff=1e-2)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=1.0))
    cfg.bridge.load_weights(tr.models, ckpt)
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    dp, dp_rank = ps.get_world_size('dp'), ps.get_rank_in('dp') if ps.get_world_size('dp') > 1 else 0
    ds = SyntheticPackedDataset(512, 128, seg_lo=16, seg_hi=64, seed=3, pin=False, segment_multiple=4)
    losses = []
    for _ in range(2):
        mbs = [ds.next_microbatch() for _ in range(4)]
        losses.append(tr.train_step(mbs[dp_rank::dp]))
    return losses, {k: v.clone() for k, v in cfg.bridge.export_weights(tr.models)}


_SINGLE = {}


def _check_layout(tmp_path, tp=1, ep=1, cp=1, pp=1):
    from dist_utils import run_ranks
    cfg, model = _model()
    d = str(tmp_path / 'ckpt')
    cfg.bridge.save_weights([model], d)
    if 'base' not in _SINGLE:
        _SINGLE['base'] = run_ranks(_train_worker, 1, d, 1, 1, 1)[0]
    base_losses, base_w = _SINGLE['base']
    for losses, weights in run_ranks(_train_worker, 4, d, tp, ep, cp, pp):
        for a, b in zip(losses, base_losses):
            assert abs(a - b) < 3e-5, (losses, base_losses)
        assert set(weights) == set(base_w)
        for k, v in base_w.items():
            assert torch.allclose(weights[k].float(), v.float(), rtol=0, atol=3e-6), \
                (k, (weights[k].float() - v.float()).abs().max().item())


def test_tp2_sequence_parallel_dp2_matches_single_process(tmp_path):
    """Query heads, sinks and output groups split over two ranks; the shared key / value head replicated."""
    _check_layout(tmp_path, tp=2)


def test_cp2_ep2_matches_single_process(tmp_path):
    """Window + sink attention over zig-zag chunks, hash routing on this rank's token ids, experts over two ranks."""
    _check_layout(tmp_path, cp=2, ep=2)


def test_lora_adapter_round_trip_uses_disk_names(tmp_path):
    import json
    import os

    from safetensors.torch import load_file

    from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
    cfg, model = _model()
    lc = LoraConfig(r=4, lora_alpha=8, target_modules='all-linear')
    peft = get_peft_model(model, lc)
    g = torch.Generator().manual_seed(7)
    with torch.no_grad():
        for n, p in sorted(peft.named_parameters(), key=lambda kv: kv[0]):
            if 'lora_' in n:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    d = str(tmp_path / 'adapter')
    cfg.bridge.save_weights([peft], d, peft_format=True)
    saved = load_file(os.path.join(d, 'adapter_model.safetensors'))
    pre = 'base_model.model.layers.0.'
    for key in ('attn.wq_a.lora_A.weight', 'attn.wq_b.lora_B.weight', 'attn.wkv.lora_A.weight',
                'attn.wo_b.lora_B.weight', 'ffn.experts.1.w1.lora_A.weight', 'ffn.experts.1.w2.lora_B.weight',
                'ffn.shared_experts.w3.lora_B.weight'):
        assert pre + key in saved, key
    assert not any('.model.model.' in k or 'gate_proj' in k for k in saved)
    ac = json.load(open(os.path.join(d, 'adapter_config.json')))
    assert {'wq_a', 'wq_b', 'wkv', 'wo_b', 'w1', 'w2', 'w3'} <= set(ac['target_modules'])
    cfg2, model2 = _model()
    peft2 = get_peft_model(model2, lc)
    cfg2.bridge.load_weights([peft2], d, peft_format=True)
    again = dict(cfg2.bridge.export_weights([peft2], peft_format=True))
    assert sorted(again) == sorted(saved) and all(torch.equal(again[k], saved[k]) for k in saved)
    ids = torch.randint(0, 512, (1, 24), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        assert torch.equal(peft.eval()(ids), peft2.eval()(ids))


def test_pp2_tp2_matches_single_process(tmp_path):
    """The streams of the hyper-connections cross the stage boundary; the hash-routed layer sits on the first stage, the
    streams' output contraction on the last; the checkpoint walk agrees across stages on which layers route by hash."""
    _check_layout(tmp_path, tp=2, pp=2)

