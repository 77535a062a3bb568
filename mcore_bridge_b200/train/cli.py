"""Command-line training entry point (``python -m mcore_bridge_b200.train.cli`` or, once installed,
``mcb200-train``); one process per GPU under ``torchrun``, or a single process.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \\
        -m mcore_bridge_b200.train.cli --model /path/to/hf_checkpoint --tp 8 --sequence-parallel \\
        --seq-len 8192 --global-batch 64 --micro-batch-size 4 --steps 100 --save /path/to/out

The reference leaves training to an external trainer (``README.md:160``); this is the in-tree equivalent built on
``Trainer.train_step``.  ``--model`` is a Hugging Face checkpoint directory (config and, unless ``--random-init``,
weights are read from it) or the name of a preset of ``train/presets.py``.  Data: ``--data`` names a ``.npy`` / ``.bin``
file of token ids (``--data-dtype``, default int32) that is cut into sequences of ``--seq-len`` tokens; without it the
run uses synthetic packed sequences.  ``--resume`` continues from a directory written by ``--save`` (optimizer state,
step, RNG); model weights are always exchanged in Hugging Face safetensors format.
"""
from __future__ import annotations

import argparse
import json
import os
import time
from typing import Dict, Iterator, List

import torch


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split('\n')[0])
    ap.add_argument('--model', required=True, help='Hugging Face checkpoint directory or preset name')
    ap.add_argument('--random-init', action='store_true', help='do not load weights from --model')
    ap.add_argument('--tp', type=int, default=1)
    ap.add_argument('--pp', type=int, default=1)
    ap.add_argument('--vpp', type=int, default=None)
    ap.add_argument('--cp', type=int, default=1)
    ap.add_argument('--ep', type=int, default=1)
    ap.add_argument('--etp', type=int, default=None)
    ap.add_argument('--sequence-parallel', action='store_true')
    ap.add_argument('--seq-len', type=int, default=4096)
    ap.add_argument('--global-batch', type=int, default=8, help='sequences per optimizer step over all ranks')
    ap.add_argument('--micro-batch-size', type=int, default=1, help='sequences per micro-batch')
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--lr', type=float, default=1e-4)
    ap.add_argument('--weight-decay', type=float, default=0.1)
    ap.add_argument('--clip-grad', type=float, default=1.0)
    ap.add_argument('--dtype', default='bf16', choices=['bf16', 'fp32'])
    ap.add_argument('--recompute-layers', type=int, default=0, help='leading layers that recompute their activations')
    ap.add_argument('--lora-rank', type=int, default=0)
    ap.add_argument('--lora-alpha', type=int, default=0, help='default: 2 x rank')
    ap.add_argument('--lora-target', default='all-linear')
    ap.add_argument('--data', default=None, help='file of token ids (.npy or raw binary)')
    ap.add_argument('--data-dtype', default='int32')
    ap.add_argument('--seed', type=int, default=1234)
    ap.add_argument('--save', default=None, help='directory for the final weights (HF format) and the training state')
    ap.add_argument('--save-interval', type=int, default=0)
    ap.add_argument('--resume', default=None)
    ap.add_argument('--log-interval', type=int, default=1)
    ap.add_argument('--heartbeat-dir', default=None)
    ap.add_argument('--overlap-param-gather', action='store_true',
                    help='overlap the parameter all-gather of a step with the forward pass of the next one')
    ap.add_argument('--set', dest='overrides', action='append', default=[], metavar='FIELD=VALUE',
                    help='any other ModelConfig field, value in Python / JSON syntax (repeatable), e.g. '
                    "--set cp_comm_type=allgather --set cpu_offloading=true --set offload_modules='[\"core_attn\"]'")
    return ap.parse_args(argv)


def parse_overrides(items) -> Dict[str, object]:
    """``FIELD=VALUE`` strings -> dict; values are read as JSON (``true``, ``3``, ``[1, 2]``, ``"text"``), then as a
    Python literal, and kept as plain text when they are neither."""
    import ast
    import json
    out = {}
    for item in items or []:
        if '=' not in item:
            raise ValueError(f'--set expects FIELD=VALUE, got {item!r}')
        key, text = item.split('=', 1)
        key = key.strip().replace('-', '_')
        try:
            val = json.loads(text)
        except ValueError:
            try:
                val = ast.literal_eval(text)
            except (ValueError, SyntaxError):
                val = text
        out[key] = val
    return out


def _hf_config(model: str):
    if os.path.isdir(model):
        from transformers import AutoConfig
        return AutoConfig.from_pretrained(model, trust_remote_code=False)
    from .presets import hf_config
    return hf_config(model)


class TokenFileDataset:
    """Sequences of ``seq_len + 1`` consecutive tokens from a flat token file; every data-parallel rank reads a
    disjoint, strided set of windows.  Yields the micro-batch dict ``Trainer.train_step`` takes."""

    def __init__(self, path: str, dtype: str, seq_len: int, micro_batch_size: int, dp_rank: int, dp_size: int):
        import numpy as np
        arr = np.load(path, mmap_mode='r') if path.endswith('.npy') else \
            np.memmap(path, dtype=np.dtype(dtype), mode='r')
        self.tokens = arr.reshape(-1)
        self.seq_len, self.mbs = seq_len, micro_batch_size
        self.n_windows = (len(self.tokens) - 1) // seq_len
        if self.n_windows < 1:
            raise ValueError(f'{path} holds fewer than {seq_len + 1} tokens')
        self.cursor, self.stride = dp_rank, dp_size

    def skip(self, n_microbatches: int) -> None:
        """Moves past ``n_microbatches`` micro-batches without reading them (resume)."""
        self.cursor += n_microbatches * self.mbs * self.stride

    def next_microbatch(self) -> Dict[str, torch.Tensor]:
        import numpy as np
        rows = []
        for _ in range(self.mbs):
            w = self.cursor % self.n_windows
            self.cursor += self.stride
            rows.append(np.asarray(self.tokens[w * self.seq_len:(w + 1) * self.seq_len + 1]).astype('int64'))
        T = self.seq_len * self.mbs
        ids = torch.from_numpy(np.concatenate([r[:-1] for r in rows]))[None]
        labels = torch.from_numpy(np.concatenate([r[1:] for r in rows]))[None]
        cu = torch.arange(0, T + 1, self.seq_len, dtype=torch.int32)
        pos = torch.arange(self.seq_len).repeat(self.mbs)[None]
        pin = torch.cuda.is_available()
        out = {'input_ids': ids, 'labels': labels, 'position_ids': pos, 'loss_mask': torch.ones(1, T),
               'cu_seqlens': cu, 'max_seqlen': self.seq_len}
        return {k: (v.pin_memory() if pin and isinstance(v, torch.Tensor) else v) for k, v in out.items()}


def main(argv=None) -> int:
    args = parse_args(argv)
    import torch.distributed as dist

    from .. import ModelConfig, get_mcore_model, hf_to_mcore_config
    from ..parallel import state as ps
    from ..utils.logger import get_logger
    from .checkpoint import load_training_state, save_training_state
    from .data import SyntheticPackedDataset
    from .trainer import TrainConfig, Trainer, init_weights
    logger = get_logger()
    ps.init_distributed()
    ps.initialize_model_parallel(tensor_model_parallel_size=args.tp, pipeline_model_parallel_size=args.pp,
                                 virtual_pipeline_model_parallel_size=args.vpp, context_parallel_size=args.cp,
                                 expert_model_parallel_size=args.ep, expert_tensor_parallel_size=args.etp)
    rank = dist.get_rank() if dist.is_initialized() else 0
    kw = hf_to_mcore_config(_hf_config(args.model))
    kw.update(tensor_model_parallel_size=args.tp, pipeline_model_parallel_size=args.pp,
              virtual_pipeline_model_parallel_size=args.vpp, context_parallel_size=args.cp,
              expert_model_parallel_size=args.ep, sequence_parallel=args.sequence_parallel and args.tp > 1)
    if args.etp is not None:
        kw['expert_tensor_parallel_size'] = args.etp
    if args.dtype == 'bf16':
        kw['bf16'] = True
    else:
        kw['params_dtype'] = torch.float32
    if args.recompute_layers > 0:
        kw.update(recompute_granularity='full', recompute_method='block', recompute_num_layers=args.recompute_layers)
    extra = parse_overrides(args.overrides)
    unknown = [k for k in extra if k not in ModelConfig.__dataclass_fields__]
    if unknown:
        raise SystemExit(f'--set: unknown ModelConfig field(s) {unknown}')
    kw.update(extra)
    cfg = ModelConfig(**kw)
    tc = TrainConfig(lr=args.lr, weight_decay=args.weight_decay, clip_grad=args.clip_grad, init_seed=args.seed,
                     heartbeat_dir=args.heartbeat_dir, overlap_param_gather=args.overlap_param_gather)
    models = get_mcore_model(cfg)
    if os.path.isdir(args.model) and not args.random_init:
        cfg.bridge.load_weights(models, args.model)
    else:
        for i, m in enumerate(models):
            init_weights(m, tc.init_std, args.seed + i)
    if args.lora_rank > 0:
        from ..tuners import LoraConfig, get_peft_model
        target = args.lora_target if args.lora_target == 'all-linear' else args.lora_target.split(',')
        lc = LoraConfig(r=args.lora_rank, lora_alpha=args.lora_alpha or 2 * args.lora_rank, target_modules=target)
        models = [get_peft_model(m, lc) for m in models]
    trainer = Trainer(cfg, tc, models=models)
    start_step = 0
    if args.resume:
        start_step = int(load_training_state(trainer, args.resume).get('step', 0))
    dp = ps.get_world_size('dp')
    dp_rank = ps.get_rank_in('dp') if dp > 1 else 0
    if args.global_batch % (dp * args.micro_batch_size):
        raise SystemExit(f'--global-batch must be a multiple of dp x micro-batch-size = {dp * args.micro_batch_size}')
    n_micro = args.global_batch // dp // args.micro_batch_size
    if args.data:
        ds = TokenFileDataset(args.data, args.data_dtype, args.seq_len, args.micro_batch_size, dp_rank, dp)
    else:
        ds = SyntheticPackedDataset(cfg.padded_vocab_size, args.seq_len, micro_batch_size=args.micro_batch_size,
                                    seed=args.seed + dp_rank, segment_multiple=max(1, args.tp * 2 * args.cp))
    if start_step:
        # continue the data stream where the interrupted run stopped
        if hasattr(ds, 'skip'):
            ds.skip(start_step * n_micro)
        else:
            for _ in range(start_step * n_micro):
                ds.next_microbatch()
    tokens_per_step = args.global_batch * args.seq_len
    t_last = time.perf_counter()
    for step in range(start_step, args.steps):
        loss = trainer.train_step([ds.next_microbatch() for _ in range(n_micro)])
        if rank == 0 and (step + 1) % args.log_interval == 0:
            now = time.perf_counter()
            rec = {'step': step + 1, **{k: round(v, 6) for k, v in trainer.last_metrics.items()},
                   'tokens_per_s': round(tokens_per_step * args.log_interval / (now - t_last), 1)}
            t_last = now
            logger.info(json.dumps(rec))
        if args.save and args.save_interval and (step + 1) % args.save_interval == 0 and step + 1 < args.steps:
            save_training_state(trainer, os.path.join(args.save, 'state'), step + 1)
    trainer.optimizer.finish_param_gather()
    if args.save:
        cfg.bridge.save_weights(trainer.models, args.save, peft_format=args.lora_rank > 0)
        save_training_state(trainer, os.path.join(args.save, 'state'), args.steps)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == '__main__':
    raise SystemExit(main())
