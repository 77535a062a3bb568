"""Worker (single process or torchrun): the fused MoE layer path (router kernel, pull dispatch over peer memory, combine)
against the torch.distributed path of the same layer, forward and backward, expert parallel over all ranks."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch.distributed as dist
from mcore_bridge_b200.parallel import state as ps
from mcore_bridge_b200.ops import _lib, moe as moe_ops
ps.init_distributed()
world = dist.get_world_size() if dist.is_initialized() else 1
rank = dist.get_rank() if dist.is_initialized() else 0
ps.initialize_model_parallel(expert_model_parallel_size=world)
dev = torch.device('cuda', torch.cuda.current_device())
from mcore_bridge_b200 import ModelConfig
from mcore_bridge_b200.train.presets import hf_config
from mcore_bridge_b200.config import hf_to_mcore_config
from mcore_bridge_b200.layers.moe import MoELayer
def rel(a,b): return ((a.float()-b.float()).norm()/(b.float().norm()+1e-9)).item()
ok = True
for (E,k,H,F,sig,groups,use_mask) in [(8,2,256,128,False,None,False),(128,8,2048,768,False,None,False),(64,6,1024,256,True,8,False),
                                      (8,2,256,128,False,None,True),(64,6,1024,256,True,8,True)]:
    kw = hf_to_mcore_config(hf_config('qwen3_moe_tiny', num_experts=E, num_experts_per_tok=k, hidden_size=H, moe_intermediate_size=F))
    if sig: kw.update(moe_router_score_function='sigmoid', moe_router_enable_expert_bias=True, moe_router_num_groups=groups, moe_router_group_topk=4, moe_router_topk_scaling_factor=2.5)
    cfg = ModelConfig(**kw, bf16=True, expert_model_parallel_size=world, moe_aux_loss_coeff=1e-2)
    torch.manual_seed(5)
    with torch.device(dev):
        layer = MoELayer(cfg).train()
    # same router on every rank; experts differ per rank (global expert e = rank*El + local)
    g = torch.Generator(device=dev).manual_seed(11)
    with torch.no_grad():
        layer.router.weight.copy_(torch.randn(layer.router.weight.shape, device=dev, generator=g)*0.3)
        if sig: layer.router.expert_bias.copy_(torch.randn(E, device=dev, generator=g)*0.05)
        full1 = torch.randn(E, layer.experts.linear_fc1.weight.shape[1], H, device=dev, generator=g)*0.05
        full2 = torch.randn(E, H, layer.experts.linear_fc2.weight.shape[2], device=dev, generator=g)*0.05
        El = E // world
        layer.experts.linear_fc1.weight.copy_(full1[rank*El:(rank+1)*El]); layer.experts.linear_fc2.weight.copy_(full2[rank*El:(rank+1)*El])
    T = 1024
    gx = torch.Generator(device=dev).manual_seed(100+rank)
    x = (torch.randn(T, H, device=dev, generator=gx)).to(torch.bfloat16)
    # padded tokens are routed like the others but stay out of the load statistics
    mask = (torch.rand(T, device=dev, generator=gx) < 0.1) if use_mask else None
    outs = {}
    # 's': exchange fused into the expert GEMMs in both directions (gather before the first, scatter after the last);
    # '1': gather fused, results pulled by the combine kernel; 'k': the separate dispatch / combine kernels;
    # '0': torch.distributed
    for fused in ('s','1','k','0'):
        os.environ['MCB200_FUSED_MOE'] = '0' if fused == '0' else '1'
        os.environ['MCB200_MOE_FUSED_GEMM'] = '0' if fused == 'k' else '1'
        os.environ['MCB200_MOE_SCATTER'] = '1' if fused == 's' else '0'
        layer.zero_grad()
        xx = x.clone().requires_grad_()
        y = layer(xx, padding_mask=mask)
        gy = torch.Generator(device=dev).manual_seed(200+rank)
        dy = torch.randn(y.shape, device=dev, generator=gy).to(torch.bfloat16)
        y.backward(dy)
        outs[fused] = (y.detach().clone(), xx.grad.clone(), layer.router.weight.grad.clone(), layer.experts.linear_fc1.weight.grad.clone(), layer.experts.linear_fc2.weight.grad.clone())
        torch.cuda.synchronize(); _lib.check_status()
    names = ['y','dx','drouter','dfc1','dfc2']
    for tag in ('s', '1', 'k'):
        for n_, a_, b_ in zip(names, outs[tag], outs['0']):
            r = rel(a_, b_); good = r < 3e-2
            t = torch.tensor([0 if good else 1], device=dev)
            if world>1: dist.all_reduce(t)
            ok &= t.item()==0
            if rank==0: print(f'E{E} k{k} H{H} sig{sig} mask{int(use_mask)} mode {tag}: {n_} rel={r:.3e} {"OK" if t.item()==0 else "FAIL"}', flush=True)
    # the row assignment of the fused dispatch+GEMM path has no atomics: a second run gives the same bits
    from mcore_bridge_b200.layers import moe_fused
    if moe_fused.pull_gemm_supported(layer.experts, layer.config, E // world, H):
        os.environ['MCB200_FUSED_MOE'] = '1'; os.environ['MCB200_MOE_FUSED_GEMM'] = '1'; os.environ['MCB200_MOE_SCATTER'] = '0'
        layer.zero_grad(); xx = x.clone().requires_grad_(); y2 = layer(xx, padding_mask=mask); y2.backward(dy)
        same = torch.equal(y2, outs['1'][0]) and torch.equal(layer.experts.linear_fc1.weight.grad, outs['1'][3])
        t = torch.tensor([0 if same else 1], device=dev)
        if world>1: dist.all_reduce(t)
        ok &= t.item()==0
        if rank==0: print(f'E{E} k{k} H{H} sig{sig}: fused path reproducible {"OK" if t.item()==0 else "FAIL"}', flush=True)
# micro-batches of different lengths reuse (and, when larger, grow) one allocation per layer shape
from mcore_bridge_b200.layers import moe_fused as _mf
kw = hf_to_mcore_config(hf_config('qwen3_moe_tiny', num_experts=8, num_experts_per_tok=2, hidden_size=256, moe_intermediate_size=128))
cfg = ModelConfig(**kw, bf16=True, expert_model_parallel_size=world)
torch.manual_seed(5)
with torch.device(dev):
    layer = MoELayer(cfg).train()
g = torch.Generator(device=dev).manual_seed(12)
with torch.no_grad():
    layer.router.weight.copy_(torch.randn(layer.router.weight.shape, device=dev, generator=g) * 0.3)
    for w in (layer.experts.linear_fc1.weight, layer.experts.linear_fc2.weight):
        w.copy_(torch.randn(w.shape, device=dev, generator=g) * 0.05)
_mf._BUFFERS.clear()
for T in (512, 256, 768, 384):
    gx = torch.Generator(device=dev).manual_seed(300 + rank + T)
    x = torch.randn(T, 256, device=dev, generator=gx).to(torch.bfloat16)
    dy = torch.randn(T, 256, device=dev, generator=gx).to(torch.bfloat16)
    res = {}
    for fused in ('1', '0'):
        os.environ['MCB200_FUSED_MOE'] = fused; os.environ['MCB200_MOE_FUSED_GEMM'] = '1'; os.environ['MCB200_MOE_SCATTER'] = '0'
        layer.zero_grad(); xx = x.clone().requires_grad_(); y = layer(xx); y.backward(dy)
        res[fused] = (y.detach().clone(), xx.grad.clone())
    torch.cuda.synchronize(); _lib.check_status()
    r = max(rel(res['1'][0], res['0'][0]), rel(res['1'][1], res['0'][1]))
    t = torch.tensor([0 if r < 3e-2 else 1], device=dev)
    if world>1: dist.all_reduce(t)
    ok &= t.item()==0
    if rank==0: print(f'varying T={T}: rel={r:.3e} allocations={len(_mf._BUFFERS)} {"OK" if t.item()==0 else "FAIL"}', flush=True)
ok &= len(_mf._BUFFERS) == 2        # one forward and one backward allocation for the layer shape
if rank==0: print('ALL OK' if ok else 'SOME FAILED', flush=True)
if world>1:
    dist.barrier(); dist.destroy_process_group()
