"""Headline benchmark: training tokens/s of a Qwen3-8B-shaped dense model, bf16, TP = N + sequence parallel,
packed 8192-token sequences, on N GPUs of one node (weak scaling: 8 packed sequences per GPU per step, so
N = 8 runs the global batch of 64 the baseline config names).

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with the step's inputs
already on the device; ``e2e`` times the same steps through ``Trainer.train_step`` from pinned host batches
with the loss read back every step.  ``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--model', default='qwen3_8b')
    ap.add_argument('--seq-len', type=int, default=8192)
    ap.add_argument('--seqs-per-gpu', type=int, default=8, help='packed sequences per GPU per step (weak scaling)')
    ap.add_argument('--layers', type=int, default=None, help='debug only: override the layer count (marks the run invalid)')
    ap.add_argument('--parallelism', default='tp', choices=['tp', 'dp', 'ep'],
                    help="'ep': expert parallel over all GPUs with data parallel dense parameters (MoE models)")
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--lora-rank', type=int, default=0,
                    help='train LoRA adapters (alpha = 2 * rank) on all linear layers with the base weights frozen')
    ap.add_argument('--recompute-layers', type=int, default=-1,
                    help='how many leading layers recompute their activations (default: none)')
    ap.add_argument('--micro-batch-size', type=int, default=0,
                    help='packed sequences per micro-batch (0: min(4, GPUs); one GPU keeps 1 to fit memory)')
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


def main():
    args = parse_args()
    if args.impl == 'reference':
        return reference_arm()
    os.environ.setdefault('PYTORCH_CUDA_ALLOC_CONF', 'expandable_segments:True')
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
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit('launch with torch.distributed.run for --gpus > 1')
    torch.cuda.set_device(local_rank)
    ps.init_distributed()
    tp = world if args.parallelism == 'tp' else 1
    ep = world if args.parallelism == 'ep' else 1
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, expert_model_parallel_size=ep)
    hf_over = {}
    if args.layers is not None:
        hf_over['num_hidden_layers'] = args.layers
    # One GPU holds all parameters, gradients and optimizer state (~148 GB) next to the activations of 8192 tokens;
    # with the activation-lean norm / gated-activation blocks every layer's activations fit (peak ~168 GB of 180), so
    # nothing is recomputed by default.  --recompute-layers N recomputes the first N layers.
    recompute = {}
    if tp == 1 and args.recompute_layers > 0:
        recompute = dict(recompute_granularity='full', recompute_method='block',
                         recompute_num_layers=args.recompute_layers)
    extra = {}
    if ep > 1 or args.parallelism == 'ep':
        extra = dict(expert_model_parallel_size=ep, moe_aux_loss_coeff=1e-3, moe_router_load_balancing_type='aux_loss')
        recompute = {}
        if args.recompute_layers > 0:
            recompute = dict(recompute_granularity='full', recompute_method='block',
                             recompute_num_layers=args.recompute_layers)
    if args.lora_rank > 0:
        recompute = {}          # frozen base weights carry no gradient or optimizer state: everything fits
    cfg = model_config(args.model, hf_over, bf16=True, tensor_model_parallel_size=tp, sequence_parallel=tp > 1,
                       **recompute, **extra)
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
    mbs = args.micro_batch_size or (8 if world >= 8 else min(4, world))
    global_batch = args.seqs_per_gpu * world
    n_micro = global_batch // dp // mbs                # micro-batches this rank runs per step
    assert n_micro * mbs * dp == global_batch
    ds = SyntheticPackedDataset(cfg.padded_vocab_size, args.seq_len, micro_batch_size=mbs,
                                seed=1234 + ps.get_rank_in('dp'), segment_multiple=max(1, tp))
    tokens_per_step = global_batch * args.seq_len

    def host_batches():
        return [ds.next_microbatch() for _ in range(n_micro)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (untimed)
    for _ in range(args.warmup):
        trainer.train_step(host_batches())
    barrier()

    # ---- device-timed region: inputs staged on the device before the clock starts
    staged = [[{k: (v.cuda(non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in mb.items()}
               for mb in host_batches()] for _ in range(args.steps)]
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.LAUNCHES
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for s in range(args.steps):
        trainer.train_step(staged[s])
    end.record()
    barrier()
    launches = _lib.LAUNCHES - launches0
    ms = start.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device='cuda')
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    del staged

    # ---- end to end: pinned host batches copied in every step, loss read back every step
    e2e = None
    if not args.no_e2e:
        batches = [host_batches() for _ in range(args.steps)]
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        barrier()
        t0 = time.perf_counter()
        for s in range(args.steps):
            trainer.train_step(batches[s])
        barrier()
        dt = time.perf_counter() - t0
        t = torch.tensor([dt], dtype=torch.float64, device='cuda')
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {'value': tokens_per_step * args.steps / float(t.item()), 'unit': 'tokens/s',
               'h2d_bytes_per_step': trainer.h2d_bytes // args.steps, 'd2h_bytes_per_step': trainer.d2h_bytes // args.steps,
               'timer': 'host wall clock between device synchronisations, max over ranks'}
    _lib.check_status()
    if rank == 0:
        out = {
            'metric': ('train tokens/s (device-timed, max over ranks) Qwen3-30B-A3B EP=N, DP=N dense, seq 4096'
                       if args.parallelism == 'ep' else
                       'train tokens/s (device-timed, max over ranks) Qwen3-8B TP=N + SP, packed 8192'),
            'value': value, 'unit': 'tokens/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
            'dtype': 'bf16', 'data': 'synthetic (uniform-random token ids, packed segments 256-4096, random-init weights)',
            'impl': 'ours',
            'config': {'model': args.model + ('' if args.layers is None else f'[layers={args.layers}: INVALID debug run]'),
                       'global_batch': global_batch, 'seq_len': args.seq_len,
                       'parallelism': (f'ep{ep} dp{dp}' if args.parallelism == 'ep' else
                                       f'tp{tp}' + ('+sp' if tp > 1 else '') + (f' dp{dp}' if dp > 1 else '')),
                       'micro_batches_per_step': n_micro, 'micro_batch_size': mbs, 'recompute': (f"full, first {recompute['recompute_num_layers']} layers" if recompute else 'none'),
                       'peak_memory_gb': round(torch.cuda.max_memory_allocated() / 2**30, 1),
                       'tp_collectives': 'fused in-kernel (NVLink peer memory)' if (tp > 1 and os.environ.get('MCB200_FUSED_COMM', '1') != '0') else ('nccl' if tp > 1 else 'none'),
                       'optimizer': 'AdamW, fp32 master weights and moments, fp32 gradient accumulation',
                       'lora': (f'rank {args.lora_rank}, alpha {2 * args.lora_rank}, all linear layers'
                                if args.lora_rank > 0 else None),
                       'l2': 'working set per step (parameters, gradients, optimizer state: > 100 GB) exceeds the 126 MB L2; no flush needed',
                       'loss': trainer.last_metrics.get('loss')},
            'clocks': clocks, 'e2e': e2e, 'gpu_launches': launches,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == '__main__':
    sys.exit(main())
