"""Kernel micro-benchmarks: ``python -m mcore_bridge_b200.bench_ops <op> [--m ..] [--n ..] [--k ..]``.

Times one in-tree kernel with CUDA events after warm-up (inputs larger than L2 where the op is memory-bound, or an
L2 flush between iterations) and prints achieved TFLOP/s or GB/s next to the measured peaks in
``MEASURED_PEAKS.json`` when that file is present.  The same command line (small sizes, few iterations) is what
the profiler captures in ``profiles/`` were taken with.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        d = json.load(open(p))
        return (d.get('bf16_tflops', 1590.0), d.get('bf16_tflops_sustained', 1400.0), d.get('hbm_gbs', 6650.0),
                'measured')
    return 1590.0, 1400.0, 6650.0, 'fallback'


def _time(fn, iters, flush=None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters * 1e-3


def step_profile(a):
    """Per-kernel device time of one ``Trainer.train_step`` (torch.profiler / kineto, CUDA activity) on a model of
    reduced depth, after three warm-up steps: the table the step-breakdown summaries under ``profiles/`` are made of.
    One GPU, or under ``torch.distributed.run`` with ``--parallelism tp`` / ``ep`` over all ranks (rank 0 reports);
    per-layer figures carry over to the full model."""
    from torch.profiler import ProfilerActivity, profile

    from .train.data import SyntheticPackedDataset
    from .train.presets import model_config
    from .train.trainer import TrainConfig, Trainer
    import os

    import torch.distributed as dist

    from .parallel import state as ps
    world, rank = int(os.environ.get('WORLD_SIZE', '1')), int(os.environ.get('RANK', '0'))
    torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
    extra = {}
    if world > 1:      # torchrun: tensor parallel (+ sequence parallel) or expert parallel over all ranks
        ps.init_distributed()
        tp = world if a.parallelism == 'tp' else 1
        ep = world if a.parallelism == 'ep' else 1
        ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep)
        extra = dict(tensor_model_parallel_size=tp, sequence_parallel=tp > 1, expert_model_parallel_size=ep)
    cfg = model_config(a.model, {'num_hidden_layers': a.layers}, bf16=True, **extra)
    tr = Trainer(cfg, TrainConfig())
    ds = SyntheticPackedDataset(cfg.padded_vocab_size, a.seq_len, micro_batch_size=1, seed=1 + rank)

    def batch():
        return [ds.next_microbatch() for _ in range(a.micro_batches)]

    for _ in range(3):
        tr.train_step(batch())
    torch.cuda.synchronize()
    mbs = batch()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        tr.train_step(mbs)
        torch.cuda.synchronize()
    rows = {}
    total = 0.0
    for ev in prof.events():
        if ev.device_type.name != 'CUDA':
            continue
        t = ev.device_time if hasattr(ev, 'device_time') else ev.cuda_time
        name = ev.name.replace('void ', '').replace('(anonymous namespace)::', '').replace('mcb::', '')
        name = name.split('<')[0].split('(')[0][:70] or ev.name[:70]
        r = rows.setdefault(name, [0.0, 0])
        r[0] += t
        r[1] += 1
        total += t
    out = {'op': 'step-profile', 'model': a.model, 'layers': a.layers, 'world': world,
           'parallelism': a.parallelism if world > 1 else 'none', 'micro_batches': a.micro_batches,
           'seq_len': a.seq_len, 'gpu_ms': round(total / 1e3, 2), 'kernels': []}
    for name, (t, n) in sorted(rows.items(), key=lambda kv: -kv[1][0])[:30]:
        out['kernels'].append({'name': name, 'ms': round(t / 1e3, 3), 'share': round(t / total, 4), 'launches': n})
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('op', choices=['step-profile', 'gemm', 'gemm_nn', 'gemm_tn', 'rmsnorm', 'rmsnorm_bwd', 'swiglu',
                                  'qkv_rope', 'ce', 'adam', 'attention', 'attention_bwd', 'gemm_fp8', 'quant_fp8',
                                  'dsa_index', 'topk', 'simple_gla', 'conv1d', 'lora'])
    ap.add_argument('--m', type=int, default=8192)
    ap.add_argument('--n', type=int, default=4096)
    ap.add_argument('--k', type=int, default=4096)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--bn', type=int, default=0)
    ap.add_argument('--no-flush', action='store_true')
    ap.add_argument('--model', default='qwen3_8b', help='step-profile: preset name')
    ap.add_argument('--layers', type=int, default=6, help='step-profile: layers of the reduced model')
    ap.add_argument('--micro-batches', type=int, default=2)
    ap.add_argument('--parallelism', default='tp', choices=['tp', 'ep'], help='step-profile under torchrun')
    ap.add_argument('--seq-len', type=int, default=8192)
    a = ap.parse_args()
    if a.op == 'step-profile':
        return step_profile(a)
    from .ops import _lib, activation, cross_entropy, gemm, norm, rope
    dev = 'cuda'
    burst, sustained, hbm, src = _peaks()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    M, N, K = a.m, a.n, a.k
    res = {'op': a.op, 'm': M, 'n': N, 'k': K}
    if a.op in ('gemm', 'gemm_nn', 'gemm_tn'):
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        fn = {'gemm': lambda: gemm.mm_nt(x, w, force_bn=a.bn), 'gemm_nn': lambda: gemm.mm_nn(dy, w, force_bn=a.bn),
              'gemm_tn': lambda: gemm.mm_tn(dy, x, force_bn=a.bn)}[a.op]
        t = _time(fn, a.iters, flush)
        tf = 2.0 * M * N * K / t / 1e12
        res.update(seconds=t, tflops=tf, frac_of_burst_peak=tf / burst, peak_source=src)
    elif a.op == 'lora':
        # the adapter GEMMs of one LoRA linear (rank --bn or 16) next to its frozen base GEMMs, forward + backward
        r = a.bn or 16
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        la = torch.randn(r, K, device=dev, dtype=torch.bfloat16) * 0.02
        lb = torch.randn(N, r, device=dev, dtype=torch.bfloat16) * 0.02
        dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        dx = torch.empty(M, K, device=dev, dtype=torch.bfloat16)

        def base():
            gemm.mm_nt(x, w, out=y)
            gemm.mm_nn(dy, w, out=dx)

        def adapter():
            t = gemm.mm_nt(x, la)                               # [M, r]
            gemm.mm_nt(t, lb, out=y, accumulate=True, alpha=2.0)
            dt = gemm.mm_nn(dy, lb, alpha=2.0)                  # [M, r]
            gemm.mm_tn(dy, t, out_dtype=torch.bfloat16)         # dB [N, r]
            gemm.mm_tn(dt, x, out_dtype=torch.bfloat16)         # dA [r, K]
            gemm.mm_nn(dt, la, out=dx, accumulate=True)

        tb = _time(base, a.iters, flush)
        ta = _time(adapter, a.iters, flush)
        moved = (2 * M * K + 3 * M * N + 2 * M * K) * 2          # x, y (r+w), dy x2, x, dx (r+w)
        res.update(rank=r, seconds_base_fwd_dgrad=tb, seconds_adapter_6_gemms=ta, adapter_over_base=ta / tb,
                   adapter_gbs=moved / ta / 1e9, frac_of_hbm_peak=moved / ta / 1e9 / hbm, peak_source=src)
    elif a.op == 'rmsnorm':
        x = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        w = torch.ones(N, device=dev, dtype=torch.bfloat16)
        t = _time(lambda: norm.rmsnorm(x, w, 1e-6), a.iters, flush)
        gbs = 2 * x.numel() * 2 / t / 1e9
        res.update(seconds=t, gbs=gbs, frac_of_hbm_peak=gbs / hbm, peak_source=src)
    elif a.op == 'rmsnorm_bwd':
        x = torch.randn(M, N, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(N, device=dev, dtype=torch.bfloat16, requires_grad=True)
        y = norm.rmsnorm(x, w, 1e-6)
        g = torch.randn_like(y)
        t = _time(lambda: y.backward(g, retain_graph=True), a.iters, flush)
        gbs = 3 * x.numel() * 2 / t / 1e9
        res.update(seconds=t, gbs=gbs, frac_of_hbm_peak=gbs / hbm, peak_source=src,
                   note='includes autograd overhead and the gradient accumulation into x.grad')
    elif a.op == 'swiglu':
        x = torch.randn(M, 2 * N, device=dev, dtype=torch.bfloat16)
        t = _time(lambda: activation.swiglu(x), a.iters, flush)
        gbs = 3 * M * N * 2 / t / 1e9
        res.update(seconds=t, gbs=gbs, frac_of_hbm_peak=gbs / hbm, peak_source=src)
    elif a.op == 'qkv_rope':
        ng, qpg, d = 8, 4, 128
        x = torch.randn(M, ng * (qpg + 2) * d, device=dev, dtype=torch.bfloat16)
        wq = torch.ones(d, device=dev, dtype=torch.bfloat16)
        ang = torch.rand(M, d // 2, device=dev)
        cos, sin = ang.cos(), ang.sin()
        t = _time(lambda: rope.qkv_split_norm_rope(x, wq, wq, cos, sin, ng, qpg, d), a.iters, flush)
        gbs = 2 * x.numel() * 2 / t / 1e9
        res.update(seconds=t, gbs=gbs, frac_of_hbm_peak=gbs / hbm, peak_source=src)
    elif a.op == 'ce':
        h = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        lab = torch.randint(0, N, (M,), device=dev)
        t = _time(lambda: cross_entropy.fused_linear_cross_entropy(h, w, lab, 'tp'), a.iters, flush)
        tf = 2.0 * M * N * K / t / 1e12
        res.update(seconds=t, tflops_forward=tf, frac_of_burst_peak=tf / burst, peak_source=src)
    elif a.op == 'attention':
        from .ops import attention as A
        nq, nkv, d = a.n // 128 if a.n >= 128 else 32, 8, 128
        q = torch.randn(M, nq, d, device=dev, dtype=torch.bfloat16)
        k = torch.randn(M, nkv, d, device=dev, dtype=torch.bfloat16)
        v = torch.randn(M, nkv, d, device=dev, dtype=torch.bfloat16)
        cu = torch.tensor([0, M], dtype=torch.int32, device=dev)
        t = _time(lambda: A.attention(q, k, v, cu, M), a.iters, flush)
        tf = 4.0 * M * M * nq * d / 2 / t / 1e12
        res.update(seconds=t, tflops_causal=tf, frac_of_burst_peak=tf / burst, heads=nq, peak_source=src)
    elif a.op == 'attention_bwd':
        from .ops import attention_cuda as AC
        nq, nkv, d = a.n // 128 if a.n >= 128 else 32, 8, 128
        seg = a.k if a.k <= M else M          # packed segments of --k tokens
        q, k, v = (torch.randn(M, h, d, device=dev, dtype=torch.bfloat16, requires_grad=True) for h in (nq, nkv, nkv))
        cu = torch.arange(0, M + 1, seg, dtype=torch.int32, device=dev)
        o = AC.attention(q, k, v, cu, seg, None)
        g = torch.randn_like(o)
        t = _time(lambda: o.backward(g, retain_graph=True), a.iters, flush)
        tf = 2.5 * 4.0 * M * seg * nq * d / 2 / t / 1e12
        res.update(seconds=t, tflops_causal=tf, frac_of_burst_peak=tf / burst, heads=nq, segment=seg, peak_source=src)
    elif a.op in ('gemm_fp8', 'quant_fp8'):
        from .ops import fp8
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        x8, sx = fp8.quantize_1x128(x)
        w8, sw = fp8.quantize_128x128(w)
        if a.op == 'gemm_fp8':
            t = _time(lambda: fp8.gemm_blockscaled(x8, sx, w8, sw), a.iters, flush)
            tf = 2.0 * M * N * K / t / 1e12
            res.update(seconds=t, tflops=tf, frac_of_bf16_burst_peak=tf / burst, peak_source=src)
        else:
            t = _time(lambda: fp8.quantize_1x128(x), a.iters, flush)
            gbs = x.numel() * 3 / t / 1e9
            res.update(seconds=t, gbs=gbs, frac_of_hbm_peak=gbs / hbm, peak_source=src)
    elif a.op in ('dsa_index', 'topk'):
        from .ops import dsa
        from .ops.attention_cuda import seq_start_from_cu
        H = 64
        q = torch.randn(M, H, 128, device=dev, dtype=torch.bfloat16)
        kk = torch.randn(M, 128, device=dev, dtype=torch.bfloat16)
        w = torch.randn(M, H, device=dev) * 0.1
        ss = seq_start_from_cu(None, M, q.device)
        if a.op == 'dsa_index':
            t = _time(lambda: dsa.index_scores_cuda(q, kk, w, ss), a.iters, flush)
            tf = 2.0 * M * M / 2 * H * 128 / t / 1e12
            res.update(seconds=t, tflops_causal=tf, frac_of_burst_peak=tf / burst, heads=H, peak_source=src,
                       note='time includes the -inf fill of the [T, T] output')
        else:
            sc = dsa.index_scores_cuda(q, kk, w, ss)
            kq = min(2048, M)
            t = _time(lambda: dsa.topk_indices(sc, kq), a.iters, flush)
            t_ref = _time(lambda: sc.topk(kq, dim=-1), max(2, a.iters // 3), flush)
            res.update(seconds=t, torch_topk_seconds=t_ref, k=kq, gbs=sc.numel() * 4 / t / 1e9)
    elif a.op == 'simple_gla':
        from .ops import gdn
        h, d = 32, 128
        seg = a.k if a.k <= M else M
        q, k, v = (torch.randn(M, h, d, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
        decay = -torch.rand(h, device=dev) * 0.1
        cu = torch.arange(0, M + 1, seg, dtype=torch.int32, device=dev)
        t = _time(lambda: gdn.simple_gla(q, k, v, decay, cu), a.iters, flush)
        o = gdn.simple_gla(q, k, v, decay, cu)
        g = torch.randn_like(o)
        tb = _time(lambda: o.backward(g, retain_graph=True), a.iters, flush)
        res.update(seconds_fwd=t, seconds_bwd=tb, heads=h, segment=seg, tokens_per_s_fwd=M / t)
    elif a.op == 'conv1d':
        from .ops import gdn
        C = N
        x = torch.randn(M, C, device=dev, dtype=torch.bfloat16, requires_grad=True)
        wc = torch.randn(C, 4, device=dev, dtype=torch.bfloat16, requires_grad=True)
        t = _time(lambda: gdn.causal_conv1d_silu(x, wc, None, None), a.iters, flush)
        gbs = 2 * x.numel() * 2 / t / 1e9
        res.update(seconds=t, gbs=gbs, frac_of_hbm_peak=gbs / hbm, peak_source=src)
    torch.cuda.synchronize()
    _lib.check_status()
    print(json.dumps(res))


if __name__ == '__main__':
    main()
