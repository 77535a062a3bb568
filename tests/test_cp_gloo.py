"""Context parallel (zig-zag chunks) on gloo ranks equals the single-process model, in loss and gradients: the ring form
(``cp_comm_type='p2p'``, one source rank per step, partial results merged through their log-sum-exp) and the all-gather
form, on two and four ranks."""
import torch

from dist_utils import run_ranks


def _batch():
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 1024, (2, 128), generator=g)
    labels = torch.randint(0, 1024, (2, 128), generator=g)
    pos = torch.arange(128).expand(2, 128).contiguous()
    return ids, labels, pos


def _worker(rank, world, ckpt_dir, packed, comm='p2p'):
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.layers.context import PackedSeqParams
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.presets import hf_config
    from mcore_bridge_b200.utils.megatron_utils import split_cp_inputs
    ps.initialize_model_parallel(context_parallel_size=world)
    cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_tiny')), params_dtype=torch.float32,
                      context_parallel_size=world, cp_comm_type=comm)
    assert model_uses(cfg, comm)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], ckpt_dir)
    ids, labels, pos = _batch()
    kw = {}
    if packed:      # the same tokens as one packed row of four sequences (lengths 64, 64, 96, 32)
        cu = torch.tensor([0, 64, 128, 224, 256], dtype=torch.int32)
        ids, labels = ids.reshape(1, -1), labels.reshape(1, -1)
        pos = torch.cat([torch.arange(int(b - a)) for a, b in zip(cu[:-1], cu[1:])]).reshape(1, -1)
        kw['packed_seq_params'] = PackedSeqParams(cu_seqlens_q=cu, cu_seqlens_kv=cu, max_seqlen_q=96, max_seqlen_kv=96)
        split = lambda t: split_cp_inputs(t, cu, 1)
    else:
        split = lambda t: split_cp_inputs(t, None, 1)
    loss = model(split(ids), position_ids=split(pos), labels=split(labels), **kw)
    (loss.sum() / labels.numel()).backward()
    gq = model.decoder.layers[0].self_attention.linear_qkv.weight.grad.clone()
    return loss.detach(), gq


def model_uses(cfg, comm):
    from mcore_bridge_b200.layers.context import layer_cp_comm_type
    return layer_cp_comm_type(cfg, 1) == (comm[0] if isinstance(comm, list) else comm)


def _reference(ckpt_dir, packed):
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.layers.context import PackedSeqParams
    from mcore_bridge_b200.train.presets import hf_config
    cfg = ModelConfig(**hf_to_mcore_config(hf_config('qwen3_tiny')), params_dtype=torch.float32)
    model = get_mcore_model(cfg)[0]
    cfg.bridge.load_weights([model], ckpt_dir)
    ids, labels, pos = _batch()
    kw = {}
    if packed:
        cu = torch.tensor([0, 64, 128, 224, 256], dtype=torch.int32)
        ids, labels = ids.reshape(1, -1), labels.reshape(1, -1)
        pos = torch.cat([torch.arange(int(b - a)) for a, b in zip(cu[:-1], cu[1:])]).reshape(1, -1)
        kw['packed_seq_params'] = PackedSeqParams(cu_seqlens_q=cu, cu_seqlens_kv=cu, max_seqlen_q=96, max_seqlen_kv=96)
    loss = model(ids, position_ids=pos, labels=labels, **kw)
    loss.mean().backward()
    return loss.detach(), model.decoder.layers[0].self_attention.linear_qkv.weight.grad.clone()


def _check(tmp_path, packed, cp=2, comm='p2p'):
    from transformers import Qwen3ForCausalLM

    from mcore_bridge_b200.train.presets import hf_config
    from mcore_bridge_b200.utils.megatron_utils import split_cp_inputs
    d = str(tmp_path / 'ckpt')
    torch.manual_seed(0)
    hf = Qwen3ForCausalLM(hf_config('qwen3_tiny')).float()
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.02) if p.dim() >= 2 else p.normal_(1.0, 0.1)
    hf.save_pretrained(d)
    ref_loss, ref_g = _reference(d, packed)
    res = run_ranks(_worker, cp, d, packed, comm)
    cu = torch.tensor([0, 64, 128, 224, 256], dtype=torch.int32) if packed else None
    for r in range(cp):
        want = split_cp_inputs(ref_loss, cu, 1, cp, r)
        assert torch.allclose(res[r][0], want, atol=1e-5), (res[r][0] - want).abs().max()
    # every rank holds the full weight; its gradient is the sum of the ranks' partial gradients
    assert torch.allclose(sum(res[r][1] for r in range(cp)), ref_g, atol=1e-6)


def test_cp2_batched(tmp_path):
    _check(tmp_path, packed=False)


def test_cp2_packed(tmp_path):
    _check(tmp_path, packed=True)


def test_cp2_packed_all_gather_form(tmp_path):
    _check(tmp_path, packed=True, comm='allgather')


def test_cp4_packed_ring(tmp_path):
    _check(tmp_path, packed=True, cp=4)


def test_cp4_batched_per_layer_comm_types(tmp_path):
    _check(tmp_path, packed=False, cp=4, comm=['p2p', 'allgather', 'p2p', 'allgather'])
