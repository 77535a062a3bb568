"""Timings of the fused compute + collective kernels against their NCCL + GEMM baselines, on the tensor-parallel
shapes of a Qwen3-8B layer.  One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \\
        -m mcore_bridge_b200.bench_comm --tokens 32768

    python -m torch.distributed.run ... -m mcore_bridge_b200.bench_comm --moe --tokens 16384   # expert parallel

``--moe`` times one Qwen3-30B-A3B MoE layer (128 experts, top-8, hidden 2048, expert FFN 768), forward + backward,
expert parallel over all ranks with ``--tokens`` tokens per rank: the exchange fused into the expert GEMMs, the
separate pull dispatch / combine kernels, and the torch.distributed all-to-all path.

Every number is device time (CUDA events) per call, max over ranks.  The roofline of a fused kernel is the slower of
its FLOPs at the measured GEMM peak and the bytes that must cross NVLink at the measured peer bandwidth.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

LINK_GBS = 770.0          # measured peer copy bandwidth per direction per GPU on this pool
GEMM_TFLOPS = 1400.0      # sustained measured cuBLAS bf16


def moe_main(a):
    import os
    from . import ModelConfig
    from .config import hf_to_mcore_config
    from .layers.moe import MoELayer
    from .ops import _lib
    from .parallel import state as ps
    from .train.presets import hf_config
    ps.init_distributed()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    ps.initialize_model_parallel(expert_model_parallel_size=world)
    dev = torch.device('cuda', torch.cuda.current_device())
    kw = hf_to_mcore_config(hf_config('qwen3_30b_a3b', num_experts=a.experts))
    cfg = ModelConfig(**kw, bf16=True, expert_model_parallel_size=world)
    torch.manual_seed(7)
    with torch.device(dev):
        layer = MoELayer(cfg).train()
    T, H = a.tokens, cfg.hidden_size
    torch.manual_seed(100 + rank)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(T, H, device=dev, dtype=torch.bfloat16)

    for p in layer.parameters():            # weight gradients accumulate into fp32 buffers, as under the trainer
        p.main_grad = torch.zeros_like(p, dtype=torch.float32)

    def step():
        layer.zero_grad(set_to_none=True)
        xx = x.detach().requires_grad_()
        layer(xx).backward(dy)

    res = {}
    for tag, fused, fgemm in (('fused_exchange_gemm', '1', '1'), ('pull_kernels', '1', '0'), ('all_to_all', '0', '0')):
        os.environ['MCB200_FUSED_MOE'] = fused
        os.environ['MCB200_MOE_FUSED_GEMM'] = fgemm
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.iters):
            step()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / a.iters], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[tag + '_us'] = round(t.item() * 1e3, 1)
        _lib.check_status()
        if a.profile:
            from torch.profiler import ProfilerActivity, profile
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(3):
                    step()
                torch.cuda.synchronize()
            if rank == 0:
                print(f'===== {tag}: device time of three iterations')
                print(prof.key_averages().table(sort_by='cuda_time_total', row_limit=20, max_name_column_width=90))
    k, F = cfg.moe_router_topk, cfg.moe_ffn_hidden_size
    flops = 3 * 2.0 * T * k * H * 3 * F          # fc1 (2F wide) + fc2, forward + two backward GEMMs each
    res['compute_us'] = round(flops / (GEMM_TFLOPS * 1e6), 1)
    # dispatch + combine, forward + backward
    res['link_us'] = round(4 * T * k * H * 2 * (world - 1) / world / (LINK_GBS * 1e3), 1)
    if rank == 0:
        print(json.dumps({'op': 'moe_layer fwd+bwd', 'ep': world, 'tokens_per_rank': T} | res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--tokens', type=int, default=8192, help='tokens of the full (gathered) micro-batch')
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--qkv', type=int, default=6144)
    ap.add_argument('--ffn', type=int, default=12288)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--moe', action='store_true', help='time the expert-parallel MoE layer instead of the TP kernels')
    ap.add_argument('--experts', type=int, default=128,
                    help='--moe: number of experts (the fused dispatch + GEMM kernel '
                    'takes at most 64 per rank, so a single-GPU run of it needs --experts 64)')
    ap.add_argument('--profile', action='store_true',
                    help='--moe: also print the per-kernel device times of three iterations (torch.profiler)')
    a = ap.parse_args()
    if a.moe:
        return moe_main(a)
    from .ops import _lib, gemm
    from .parallel import fused_comm as fc
    from .parallel import mappings as M
    from .parallel import state as ps
    ps.init_distributed()
    world, rank = dist.get_world_size(), dist.get_rank()
    ps.initialize_model_parallel(tensor_model_parallel_size=world)
    dev = torch.device('cuda', torch.cuda.current_device())
    torch.manual_seed(100 + rank)

    def bench(f):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.iters):
            f()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e3          # us

    T, H = a.tokens, a.hidden
    rows = T // world
    out = []
    for name, K, N in (('qkv', H, a.qkv // world), ('fc1', H, 2 * a.ffn // world)):
        x = torch.randn(rows, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        assert fc.enabled(x, w, 'tp'), 'fused kernels unavailable (symmetric memory)'
        t_f = bench(lambda: fc.all_gather_gemm(x, w, None, 'tp'))
        t_n = bench(lambda: gemm.mm_nt(M.all_gather_dim0(x, 'tp'), w))
        link = (world - 1) * rows * K * 2 / (LINK_GBS * 1e3)             # us
        comp = 2.0 * T * N * K / (GEMM_TFLOPS * 1e6)
        out.append(dict(op=f'ag_gemm {name}', fused_us=t_f, nccl_plus_gemm_us=t_n, link_us=link, compute_us=comp,
                        roofline_frac=max(link, comp) / t_f))
    for name, K, N in (('oproj', H // world, H), ('fc2', a.ffn // world, H)):
        xf = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        t_f = bench(lambda: fc.gemm_reduce_scatter(xf, w, 'tp'))
        t_n = bench(lambda: M.reduce_scatter_dim0(gemm.mm_nt(xf, w), 'tp'))
        link = (world - 1) * rows * N * 2 / (LINK_GBS * 1e3)
        comp = 2.0 * T * N * K / (GEMM_TFLOPS * 1e6)
        out.append(dict(op=f'gemm_rs {name}', fused_us=t_f, nccl_plus_gemm_us=t_n, link_us=link, compute_us=comp,
                        roofline_frac=max(link, comp) / t_f))
        out[-1]['gemm_only_us'] = round(bench(lambda: gemm.mm_nt(xf, w)), 1)
    torch.cuda.synchronize()
    _lib.check_status()
    if rank == 0:
        for r in out:
            print(json.dumps({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()} |
                             {'tp': world, 'tokens': T}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
