"""Headline benchmark: training tokens/s, device-timed, max over ranks, on N GPUs of one node.

Primary run (every N): Qwen3-8B-shaped dense model, bf16, TP = N + sequence parallel, packed 8192-token
sequences, weak scaling with 8 packed sequences per GPU per step (N = 8 is the global batch of 64).
Secondary run (N = 8 only, reported under ``secondary`` in the same JSON line): Qwen3-30B-A3B-shaped MoE,
EP = 8 with data-parallel dense parameters and the distributed optimizer, sequences of 4096 tokens, global
batch 128, load-balancing loss 1e-3.  On fewer GPUs the secondary entry says that the model does not fit.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with the step's inputs
already on the device; ``e2e`` times the same steps through ``Trainer.train_step`` from pinned host batches
with the loss read back every step.  With N >= 2 a self-check of the fused compute + collective kernels
against ``torch.distributed`` at the run's shapes precedes the warm-up (``selfcheck`` in the JSON line; a
mismatch makes the exit code non-zero).

``--impl reference`` reports why the reference cannot run here.  ``--impl torchlib`` runs the same trainer with
every in-tree kernel switched off (cuBLAS, flash-attn / torch attention, NCCL collectives): a library stand-in to
compare against, NOT the reference.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

TORCHLIB_ENV = {'MCB200_DISABLE_CUDA_KERNELS': '1', 'MCB200_FUSED_COMM': '0', 'MCB200_FUSED_MOE': '0',
                'MCB200_FUSED_DP': '0'}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference', 'torchlib'])
    ap.add_argument('--model', default='qwen3_8b')
    ap.add_argument('--seq-len', type=int, default=0, help='0: the model\'s benchmark length (8192 dense, 4096 MoE)')
    ap.add_argument('--seqs-per-gpu', type=int, default=0,
                    help='sequences per GPU per step, weak scaling (0: 8 for the dense model, 16 for the MoE model)')
    ap.add_argument('--layers', type=int, default=None,
                    help='debug only: override the layer count (marks the run invalid)')
    ap.add_argument('--parallelism', default='tp', choices=['tp', 'dp', 'ep'],
                    help="'ep': expert parallel over all GPUs with data parallel dense parameters (MoE models)")
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-secondary', action='store_true', help='skip the MoE run that follows the dense run at 8 GPUs')
    ap.add_argument('--secondary-steps', type=int, default=10)
    ap.add_argument('--no-selfcheck', action='store_true')
    ap.add_argument('--stage2', default=None, help=argparse.SUPPRESS)   # set by the script itself (see main)
    ap.add_argument('--lora-rank', type=int, default=0,
                    help='train LoRA adapters (alpha = 2 * rank) on all linear layers with the base weights frozen')
    ap.add_argument('--recompute-layers', type=int, default=-1,
                    help='how many leading layers recompute their activations (default: none)')
    ap.add_argument('--micro-batch-size', type=int, default=0,
                    help='sequences per micro-batch (0: chosen per model and GPU count)')
    return ap.parse_args()


def reference_arm():
    why = ('reference installs only with --no-deps and cannot be imported: its substrate megatron-core, '
           'transformer_engine and peft are not in the image or the offline wheelhouse')
    try:
        sys.path.insert(0, os.path.join(REPO, 'baseline', '_ref'))
        import mcore_bridge  # noqa: F401
        mcore_bridge.GPTBridge  # noqa: B018  (forces the lazy import that needs megatron/peft)
        why = 'reference imported, but it ships no trainer (training is delegated to ms-swift, which is absent)'
    except Exception as e:  # expected here
        why += f' ({type(e).__name__}: {str(e)[:80]})'
    if int(os.environ.get('RANK', '0')) == 0:
        print(json.dumps({'impl': 'reference', 'unavailable': why}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only queries)."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
         'clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(suffix='.csv')
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.f = open(self.path, 'w')
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '200', '-i', str(self.gpu_index)], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(',')]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'),
                                     parts[5:9]):
                    if val.lower().startswith('active'):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out['sm_mhz'] = statistics.median(sm)
            out['sm_max_mhz'] = max(mx)
            out['samples'] = len(sm)
        out['reasons'] = sorted(reasons)
        return out


def _rel(a, b):
    a, b = a.float(), b.float()
    return float(((a - b).norm() / (b.norm() + 1e-9)).item()), float((a - b).abs().max().item())


def selfcheck_tp(tokens: int, cfg) -> dict:
    """Fused AG->GEMM / GEMM->RS kernels against all_gather / reduce_scatter + the plain GEMM, at the shapes of one
    layer of the run (``tokens`` = gathered rows of a micro-batch).  Collective: every rank calls it."""
    import torch

    from mcore_bridge_b200.ops import gemm
    from mcore_bridge_b200.parallel import fused_comm as fc
    from mcore_bridge_b200.parallel import mappings as M
    from mcore_bridge_b200.parallel import state as ps
    world = ps.get_world_size('tp')
    dev = torch.device('cuda', torch.cuda.current_device())
    H = cfg.hidden_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_query_groups) * cfg.kv_channels // world
    ffn = cfg.ffn_hidden_size // world
    rows = tokens // world
    g = torch.Generator(device=dev).manual_seed(4242 + ps.get_rank_in('tp'))
    out = {}

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(torch.bfloat16)

    for name, K, N in (('qkv', H, qkv), ('fc1', H, 2 * ffn)):
        x, w = rnd(rows, K), rnd(N, K, scale=0.02)
        if not fc.enabled(x, w, 'tp'):
            return {'skipped': 'fused kernels not enabled'}
        y, xg = fc.all_gather_gemm(x, w, None, 'tp')
        xr = M.all_gather_dim0(x, 'tp')
        out[f'all_gather_gemm {name}'] = _rel(y, gemm.mm_nt(xr, w))
        out[f'all_gather_gemm {name} gathered'] = _rel(xg, xr)
        dy = rnd(tokens, N)
        out[f'gemm_reduce_scatter_nn {name}'] = _rel(fc.gemm_reduce_scatter_nn(dy, w, 'tp'),
                                                     M.reduce_scatter_dim0(gemm.mm_nn(dy, w), 'tp'))
        del x, w, y, xg, xr, dy
    for name, K, N in (('oproj', cfg.num_attention_heads * cfg.kv_channels // world, H), ('fc2', ffn, H)):
        xf, w = rnd(tokens, K), rnd(N, K, scale=0.02)
        out[f'gemm_reduce_scatter {name}'] = _rel(fc.gemm_reduce_scatter(xf, w, 'tp'),
                                                  M.reduce_scatter_dim0(gemm.mm_nt(xf, w), 'tp'))
        dy = rnd(rows, N)
        dx, _ = fc.all_gather_gemm_nn(dy, w, 'tp')
        out[f'all_gather_gemm_nn {name}'] = _rel(dx, gemm.mm_nn(M.all_gather_dim0(dy, 'tp'), w))
        del xf, w, dy, dx
    torch.cuda.synchronize()
    return out


def selfcheck_dp(numel: int = 1 << 24) -> dict:
    """Peer-memory reduce-scatter / all-gather of the distributed optimizer against torch.distributed."""
    import torch
    import torch.distributed as dist

    from mcore_bridge_b200.parallel import dp_comm
    from mcore_bridge_b200.parallel import state as ps
    dev = torch.device('cuda', torch.cuda.current_device())
    if not dp_comm.usable('dp', dev):
        return {'skipped': 'peer-memory data-parallel collectives not enabled'}
    n, r = ps.get_world_size('dp'), ps.get_rank_in('dp')
    ws, flat = dp_comm.allocate('dp', numel, torch.float32)
    g = torch.Generator(device=dev).manual_seed(99 + r)
    src = torch.randn(numel, device=dev, generator=g)
    flat.copy_(src)
    ref = torch.empty(numel // n, device=dev)
    dist.reduce_scatter_tensor(ref, src, group=ps.get_group('dp'))
    dp_comm.reduce_scatter_(ws, flat, 0, numel, 1.0)
    shard = slice(r * (numel // n), (r + 1) * (numel // n))
    out = {'dp_reduce_scatter': _rel(flat[shard], ref)}
    full = torch.empty(numel, device=dev)
    dist.all_gather_into_tensor(full, flat[shard].contiguous(), group=ps.get_group('dp'))
    dp_comm.all_gather_(ws, flat, 0, numel)
    out['dp_all_gather'] = _rel(flat, full)
    torch.cuda.synchronize()
    return out


def selfcheck_moe(cfg, tokens: int) -> dict:
    """One MoE layer of the run's shape: fused peer-memory exchange against the all-to-all path, forward and the
    input / router / expert gradients."""
    import torch

    from mcore_bridge_b200.layers.moe import MoELayer
    from mcore_bridge_b200.parallel import state as ps
    dev = torch.device('cuda', torch.cuda.current_device())
    r = ps.get_rank_in('ep')
    torch.manual_seed(77)
    with torch.device(dev):
        layer = MoELayer(cfg).train()
    g = torch.Generator(device=dev).manual_seed(11)
    with torch.no_grad():
        layer.router.weight.copy_(torch.randn(layer.router.weight.shape, device=dev, generator=g) * 0.05)
        ge = torch.Generator(device=dev).manual_seed(500 + r)
        for w in (layer.experts.linear_fc1.weight, layer.experts.linear_fc2.weight):
            w.copy_(torch.randn(w.shape, device=dev, generator=ge) * 0.03)
    gx = torch.Generator(device=dev).manual_seed(100 + r)
    x = torch.randn(tokens, cfg.hidden_size, device=dev, generator=gx).to(torch.bfloat16)
    dy = torch.randn(tokens, cfg.hidden_size, device=dev, generator=gx).to(torch.bfloat16)
    res = {}
    prev = os.environ.get('MCB200_FUSED_MOE')
    for fused in ('1', '0'):
        os.environ['MCB200_FUSED_MOE'] = fused
        layer.zero_grad()
        xx = x.clone().requires_grad_()
        y = layer(xx)
        y.backward(dy)
        res[fused] = (y.detach().clone(), xx.grad.clone(), layer.router.weight.grad.clone(),
                      layer.experts.linear_fc1.weight.grad.clone(), layer.experts.linear_fc2.weight.grad.clone())
    if prev is None:
        os.environ.pop('MCB200_FUSED_MOE', None)
    else:
        os.environ['MCB200_FUSED_MOE'] = prev
    out = {f'moe {n}': _rel(a, b) for n, a, b in zip(('y', 'dx', 'drouter', 'dfc1', 'dfc2'), res['1'], res['0'])}
    del layer, res
    torch.cuda.synchronize()
    return out


def teardown(trainer=None):
    """Releases a run's model, optimizer state, peer-mapped workspaces and process groups so that another
    configuration can be built in the same processes."""
    import torch

    from mcore_bridge_b200.layers import moe_fused
    from mcore_bridge_b200.parallel import fused_comm, symm
    from mcore_bridge_b200.parallel import state as ps
    if trainer is not None:
        trainer.optimizer = trainer.ddp = trainer.models = None
    gc.collect()
    torch.cuda.synchronize()
    moe_fused._BUFFERS.clear()
    fused_comm._ptr_cache.clear()
    symm.free_all()
    ps.destroy_model_parallel()
    gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()


def run_config(args, *, model: str, parallelism: str, steps: int, warmup: int, seq_len: int, seqs_per_gpu: int,
               mbs: int, packed: bool, tol: float = 1e-2) -> dict:
    """Builds the model under the given layout, checks the fused kernels, warms up, times ``steps`` steps on the
    device and then end to end.  Returns the result dict (the same on every rank up to rank-0-only fields)."""
    import torch
    import torch.distributed as dist

    from mcore_bridge_b200.ops import _lib
    from mcore_bridge_b200.parallel import state as ps
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    tp = world if parallelism == 'tp' else 1
    ep = world if parallelism == 'ep' else 1
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep)
    hf_over = {}
    if args.layers is not None:
        hf_over['num_hidden_layers'] = args.layers
    # One GPU holds all parameters, gradients and optimizer state (~148 GB) next to the activations of 8192 tokens;
    # with the activation-lean norm / gated-activation blocks every layer's activations fit (peak ~168 GB of 180), so
    # nothing is recomputed by default.  --recompute-layers N recomputes the first N layers.
    recompute = {}
    if args.recompute_layers > 0 and args.lora_rank == 0:
        recompute = dict(recompute_granularity='full', recompute_method='block',
                         recompute_num_layers=args.recompute_layers)
    extra = {}
    if parallelism == 'ep':
        extra = dict(expert_model_parallel_size=ep, moe_aux_loss_coeff=1e-3, moe_router_load_balancing_type='aux_loss')
    cfg = model_config(model, hf_over, bf16=True, tensor_model_parallel_size=tp, sequence_parallel=tp > 1,
                       **recompute, **extra)
    fused = args.impl == 'ours'
    selfcheck = None
    if fused and world > 1 and not args.no_selfcheck:
        selfcheck = {}
        if tp > 1:
            selfcheck.update(selfcheck_tp(mbs * seq_len, cfg))
        if ps.get_world_size('dp') > 1:
            selfcheck.update(selfcheck_dp())
        if ep > 1:
            selfcheck.update(selfcheck_moe(cfg, mbs * seq_len))
        _lib.check_status()
    models = None
    if args.lora_rank > 0:
        from mcore_bridge_b200 import get_mcore_model
        from mcore_bridge_b200.train.trainer import init_weights
        from mcore_bridge_b200.tuners import LoraConfig, get_peft_model
        tc0 = TrainConfig()
        models = get_mcore_model(cfg)
        for i, m in enumerate(models):
            init_weights(m, tc0.init_std, (tc0.init_seed or 0) + i)
        lc = LoraConfig(r=args.lora_rank, lora_alpha=2 * args.lora_rank,
                        target_modules=['linear_qkv', 'linear_proj', 'linear_fc1', 'linear_fc2'])
        models = [get_peft_model(m, lc) for m in models]
    trainer = Trainer(cfg, TrainConfig(), models=models)
    dp = ps.get_world_size('dp')
    global_batch = seqs_per_gpu * world
    n_micro = global_batch // dp // mbs                # micro-batches this rank runs per step
    assert n_micro * mbs * dp == global_batch, (global_batch, dp, mbs)
    ds = SyntheticPackedDataset(cfg.padded_vocab_size, seq_len, micro_batch_size=mbs, packed=packed,
                                seed=1234 + ps.get_rank_in('dp'), segment_multiple=max(1, tp))
    tokens_per_step = global_batch * seq_len

    def host_batches():
        return [ds.next_microbatch() for _ in range(n_micro)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (untimed)
    for _ in range(warmup):
        trainer.train_step(host_batches())
    barrier()

    # ---- device-timed region: inputs staged on the device before the clock starts
    staged = [[{k: (v.cuda(non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in mb.items()}
               for mb in host_batches()] for _ in range(steps)]
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.LAUNCHES
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for s in range(steps):
        trainer.train_step(staged[s])
    end.record()
    barrier()
    launches = _lib.LAUNCHES - launches0
    ms = start.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device='cuda')
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / steps
    value = tokens_per_step / (ms_per_step / 1e3)
    del staged

    # ---- end to end: pinned host batches copied in every step, loss read back every step
    e2e = None
    if not args.no_e2e:
        batches = [host_batches() for _ in range(steps)]
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        barrier()
        t0 = time.perf_counter()
        for s in range(steps):
            trainer.train_step(batches[s])
        barrier()
        dt = time.perf_counter() - t0
        t = torch.tensor([dt], dtype=torch.float64, device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {'value': tokens_per_step * steps / float(t.item()), 'unit': 'tokens/s',
               'h2d_bytes_per_step': trainer.h2d_bytes // steps, 'd2h_bytes_per_step': trainer.d2h_bytes // steps,
               'timer': 'host wall clock between device synchronisations, max over ranks'}
    _lib.check_status()
    moe = parallelism == 'ep'
    if packed:
        data = 'synthetic (uniform-random token ids, packed segments 256-4096, random-init weights)'
    else:
        data = f'synthetic (uniform-random token ids, unpacked sequences of {seq_len} tokens, random-init weights)'
    out = {
        'metric': ('train tokens/s (device-timed, max over ranks) Qwen3-30B-A3B EP=N, DP=N dense, seq 4096' if moe else
                   'train tokens/s (device-timed, max over ranks) Qwen3-8B TP=N + SP, packed 8192'),
        'value': value, 'unit': 'tokens/s', 'n_gpus': world, 'steps': steps, 'warmup': warmup,
        'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'bf16', 'data': data, 'impl': args.impl,
        'config': {'model': model + ('' if args.layers is None else f'[layers={args.layers}: INVALID debug run]'),
                   'global_batch': global_batch, 'seq_len': seq_len,
                   'parallelism': (f'ep{ep} dp{dp}' if moe else
                                   f'tp{tp}' + ('+sp' if tp > 1 else '') + (f' dp{dp}' if dp > 1 else '')),
                   'micro_batches_per_step': n_micro, 'micro_batch_size': mbs,
                   'recompute': (f"full, first {recompute['recompute_num_layers']} layers" if recompute else 'none'),
                   'peak_memory_gb': round(torch.cuda.max_memory_allocated() / 2**30, 1),
                   'kernels': ('in-tree sm_100a kernels' if fused else
                               'library stand-in: cuBLAS GEMMs, flash-attn / torch attention, torch element-wise ops'),
                   'collectives': (('fused in-kernel over NVLink peer memory'
                                    if os.environ.get('MCB200_FUSED_COMM', '1') != '0' else 'nccl')
                                   if world > 1 else 'none'),
                   'optimizer': 'AdamW, fp32 master weights and moments, fp32 gradient accumulation',
                   'lora': (f'rank {args.lora_rank}, alpha {2 * args.lora_rank}, all linear layers'
                            if args.lora_rank > 0 else None),
                   'l2': ('working set per step (parameters, gradients, optimizer state: > 100 GB) exceeds the 126 MB '
                          'L2; no flush needed'),
                   'loss': trainer.last_metrics.get('loss')},
        'clocks': clocks, 'e2e': e2e, 'gpu_launches': launches,
    }
    if selfcheck is not None:
        out['selfcheck'] = {k: ({'rel': round(v[0], 6), 'max_abs': round(v[1], 5)} if isinstance(v, tuple) else v)
                            for k, v in selfcheck.items()}
        bad = [k for k, v in selfcheck.items() if isinstance(v, tuple) and not (v[0] < tol)]
        out['selfcheck_failed'] = bad
    teardown(trainer)
    return out


def main():
    args = parse_args()
    if args.impl == 'reference':
        return reference_arm()
    if args.stage2:
        return stage2(args)
    if args.impl == 'torchlib':
        os.environ.update(TORCHLIB_ENV)
    os.environ.setdefault('PYTORCH_CUDA_ALLOC_CONF', 'expandable_segments:True')
    import torch
    import torch.distributed as dist

    from mcore_bridge_b200.parallel import state as ps

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if world == 1 and args.gpus > 1:
        raise SystemExit('launch with torch.distributed.run for --gpus > 1')
    torch.cuda.set_device(local_rank)
    ps.init_distributed()
    moe_primary = args.parallelism == 'ep'
    seq_len = args.seq_len or (4096 if moe_primary else 8192)
    seqs = args.seqs_per_gpu or (16 if moe_primary else 8)
    if moe_primary:
        mbs = args.micro_batch_size or 2
    else:
        mbs = args.micro_batch_size or (8 if world >= 8 else min(4, world))
    if args.impl == 'torchlib' and args.recompute_layers < 0 and world == 1:
        args.recompute_layers = 36       # the library path keeps fp32 logits and unfused activations: recompute to fit
    out = run_config(args, model=args.model, parallelism=args.parallelism, steps=args.steps, warmup=args.warmup,
                     seq_len=seq_len, seqs_per_gpu=seqs, mbs=mbs, packed=not moe_primary)
    failed = list(out.get('selfcheck_failed') or [])
    if not moe_primary and args.model == 'qwen3_8b' and not args.no_secondary and args.lora_rank == 0:
        if world >= 8:
            # The second model runs in a fresh process image: every rank parks the dense result, leaves the process
            # group and re-executes this script with --stage2.  A new image starts with empty device memory, which no
            # amount of reference dropping guarantees for 16 GB of model state plus peer-mapped workspaces per rank.
            path = _stage_path()
            if rank == 0:
                import socket
                with socket.socket() as sk:     # a free port for the second rendezvous (all ranks are on this node)
                    sk.bind(('127.0.0.1', 0))
                    port = sk.getsockname()[1]
                with open(path, 'w') as f:
                    json.dump({'port': port, 'result': out}, f)
            dist.barrier()
            dist.destroy_process_group()
            sys.stdout.flush()
            sys.stderr.flush()
            os.execv(sys.executable, [sys.executable, os.path.abspath(__file__)] + sys.argv[1:] + ['--stage2', path])
        out['secondary'] = {'model': 'qwen3_30b_a3b', 'unavailable': (
            f'does not fit on {world} GPU(s): 30.5 B parameters need 16 bytes each for bf16 weights, fp32 '
            'gradients, master weights and Adam moments (488 GB) before activations; measured at 8 GPUs (EP = 8)')}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 1 if failed else 0


def _stage_path() -> str:
    return os.path.join(tempfile.gettempdir(), f"mcb200_bench_{os.environ.get('MASTER_PORT', '0')}_stage1.json")


def stage2(args) -> int:
    """Second half of the 8-GPU run, in the re-executed processes: the Qwen3-30B-A3B EP = 8 configuration.  Rank 0
    merges it into the dense result written by the first half and prints the one JSON line."""
    os.environ.setdefault('PYTORCH_CUDA_ALLOC_CONF', 'expandable_segments:True')
    from datetime import timedelta

    import torch
    import torch.distributed as dist

    from mcore_bridge_b200.parallel import state as ps
    world, rank = int(os.environ['WORLD_SIZE']), int(os.environ['RANK'])
    with open(args.stage2) as f:
        stage1 = json.load(f)
    error = False
    try:
        torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
        # a rendezvous store of its own (rank 0 hosts it on the port chosen by the first half): the launcher's store
        # still holds the keys of the first initialisation
        store = dist.TCPStore(os.environ.get('MASTER_ADDR', '127.0.0.1'), int(stage1['port']), world,
                              is_master=(rank == 0), timeout=timedelta(seconds=600))
        ps.init_distributed(store=store)
        sec = run_config(args, model='qwen3_30b_a3b', parallelism='ep', steps=args.secondary_steps,
                         warmup=min(3, max(args.warmup, 3)), seq_len=4096, seqs_per_gpu=16, mbs=2, packed=False,
                         tol=3e-2)
    except Exception as e:      # the dense result must not be lost with the second model's run
        sec = {'model': 'qwen3_30b_a3b', 'error': f'{type(e).__name__}: {str(e)[:300]}'}
        error = True
    failed = []
    if rank == 0:
        out = stage1['result']
        os.unlink(args.stage2)
        failed = list(out.get('selfcheck_failed') or []) + list(sec.get('selfcheck_failed') or [])
        out['secondary'] = sec
        print(json.dumps(out), flush=True)
    if error:
        # the failed run may have left collectives or the CUDA context unusable: leave without the usual teardown
        sys.stderr.flush()
        os._exit(1 if failed else 0)
    dist.barrier()
    dist.destroy_process_group()
    return 1 if failed else 0


if __name__ == '__main__':
    sys.exit(main())
