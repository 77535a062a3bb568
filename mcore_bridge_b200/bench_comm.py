"""Timings of the fused compute + collective kernels against their NCCL + GEMM baselines, on the tensor-parallel
shapes of a Qwen3-8B layer.  One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \\
        -m mcore_bridge_b200.bench_comm --tokens 32768

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--tokens', type=int, default=8192, help='tokens of the full (gathered) micro-batch')
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--qkv', type=int, default=6144)
    ap.add_argument('--ffn', type=int, default=12288)
    ap.add_argument('--iters', type=int, default=20)
    a = ap.parse_args()
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
