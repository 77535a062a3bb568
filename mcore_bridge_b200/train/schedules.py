"""Pipeline-parallel micro-batch schedules over ``torch.distributed`` point-to-point (NCCL on GPUs).

* no pipelining — handled directly by ``Trainer.train_step``.
* 1F1B (one model chunk per rank): ``pp - rank - 1`` warm-up forwards, then one-forward-one-backward, then the
  cool-down backwards.  Sends are asynchronous (``isend``) and complete in the background while the next
  forward/backward runs (``overlap_p2p_comm``); receives are posted before the compute they are needed after.
* virtual pipeline (several model chunks per rank, ``virtual_pipeline_model_parallel_size``): interleaved 1F1B
  when the number of micro-batches is a multiple of the pipeline size — virtual micro-batches are walked in groups
  of ``pp`` per chunk, ``(pp - rank - 1) * 2 + (V - 1) * pp`` warm-up forwards, then one-forward-one-backward,
  then the cool-down backwards, the ordering Megatron uses — otherwise chunk by chunk (all forwards, then all
  backwards; same data flow, GPipe-like memory).  Activations and gradients travel on two communicators so that a
  pair of ranks that exchanges both (``pp = 2`` with virtual stages) never mixes them in one ordered channel.

Activations travel as ``[T_local, H]`` in ``pipeline_dtype``.  With ``variable_seq_lengths`` the shape is sent
first (two int64).  The last stage computes the loss; every stage accumulates gradients into the fp32 buffers of
the distributed optimizer exactly as in the non-pipelined path.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..layers.context import PackedSeqParams
from ..parallel import state as ps


class _P2P:

    def __init__(self, config, device):
        self.cfg, self.device = config, device
        self.prev, self.next = ps.get_pipeline_model_parallel_prev_rank(), ps.get_pipeline_model_parallel_next_rank()
        self.group = ps.get_group('pp')
        self.group_bwd = ps.get_group('pp_bwd')
        self.pending: List = []

    def _shape(self, t: Optional[torch.Tensor], peer: int, send: bool, hidden: int, default_rows: int):
        if not self.cfg.variable_seq_lengths:
            return (default_rows, hidden)
        meta = torch.zeros(2, dtype=torch.int64, device=self.device)
        if send:
            meta[0], meta[1] = t.shape[0], t.shape[1]
            self.pending.append((dist.isend(meta, peer, group=self.group), meta))  # never block the sender
            return tuple(t.shape)
        dist.recv(meta, peer, group=self.group)
        return (int(meta[0]), int(meta[1]))

    def send(self, t: torch.Tensor, peer: int, grad: bool = False):
        t = t.detach().to(self.cfg.pipeline_dtype).contiguous()
        if not grad:
            self._shape(t, peer, True, t.shape[1], t.shape[0])
        self.pending.append((dist.isend(t, peer, group=self.group_bwd if grad else self.group), t))

    def recv(self, peer: int, rows: int, hidden: int, grad: bool = False) -> torch.Tensor:
        shape = (rows, hidden) if grad else self._shape(None, peer, False, hidden, rows)
        buf = torch.empty(shape, dtype=self.cfg.pipeline_dtype, device=self.device)
        dist.recv(buf, peer, group=self.group_bwd if grad else self.group)
        return buf

    def drain(self):
        for w, _ in self.pending:
            w.wait()
        self.pending.clear()


def _psp(d: Dict):
    if d.get('cu_seqlens') is None:
        return None
    return PackedSeqParams(cu_seqlens_q=d['cu_seqlens'], cu_seqlens_kv=d['cu_seqlens'],
                           max_seqlen_q=d.get('max_seqlen'), max_seqlen_kv=d.get('max_seqlen'))


def _local_rows(d: Dict, cfg) -> int:
    rows = d['input_ids'].numel()
    if cfg.sequence_parallel and ps.get_world_size('tp') > 1:
        rows //= ps.get_world_size('tp')
    return rows


def _forward(trainer, model, d: Dict, input_tensor: Optional[torch.Tensor], n_micro: int, is_last: bool):
    cfg = trainer.config
    if input_tensor is not None:
        input_tensor.requires_grad_(True)
        inner = model.module if hasattr(model, 'module') else model
        inner.set_input_tensor(input_tensor)
    from .trainer import model_extras
    out = model(input_ids=d['input_ids'], position_ids=d.get('position_ids'), attention_mask=d.get('attention_mask'),
                labels=d['labels'] if is_last else None, packed_seq_params=_psp(d), loss_mask=d.get('loss_mask'),
                **model_extras(d))
    if is_last:
        mask = d.get('loss_mask')
        if mask is None:
            mask = torch.ones_like(out)
        ntok = mask.sum()
        if ps.get_world_size('cp') > 1:
            ntok = ntok.clone()
            dist.all_reduce(ntok, group=ps.get_group('cp'))
        # a context-parallel rank's share of the micro-batch loss, scaled by cp (see
        # Trainer.forward_backward_microbatch)
        out = (out * mask).sum() / ntok.clamp(min=1.0) * (float(ps.get_world_size('cp')) / n_micro)
    return out


def _pipeline_width(trainer) -> int:
    """Columns of the tensor sent between stages: the hidden size, or what the model declares when it sends more than
    the hidden states (Gemma-4 packs its per-layer inputs and shared keys / values behind them; with hyper-connections
    the residual streams travel side by side)."""
    m = trainer.models[0]
    m = getattr(m, 'language_model', m)
    fn = getattr(m, 'pipeline_width', None)
    if fn is not None:
        return int(fn())
    cfg = trainer.config
    if cfg.enable_hyper_connections:          # all residual streams cross the boundary side by side
        return cfg.hidden_size * int(cfg.num_residual_streams)
    return cfg.hidden_size


def _backward(output: torch.Tensor, grad: Optional[torch.Tensor], input_tensor: Optional[torch.Tensor]):
    if grad is None:
        output.backward()
    else:
        torch.autograd.backward(output, grad.to(output.dtype))
    return None if input_tensor is None else input_tensor.grad


def forward_backward_pipelining(trainer, microbatches: List[Dict]) -> torch.Tensor:
    """Runs all micro-batches through the pipeline; returns the summed (already averaged) loss on the last stage,
    zero elsewhere."""
    cfg = trainer.config
    pp, rank = ps.get_pipeline_model_parallel_world_size(), ps.get_pipeline_model_parallel_rank()
    n = len(microbatches)
    dev = trainer.device
    p2p = _P2P(cfg, dev)
    H = _pipeline_width(trainer)
    trainer.optimizer.zero_grad()
    from ..layers.mtp import MTPLossAutoScaler
    from ..ops.moe import MoEAuxLossAutoScaler
    MoEAuxLossAutoScaler.set_loss_scale(float(ps.get_world_size('cp')) / n)
    MTPLossAutoScaler.set_loss_scale(1.0 / n)
    total = torch.zeros((), dtype=torch.float32, device=dev)
    data = [trainer._prepare(mb) for mb in microbatches]
    chunks = trainer.ddp
    for m in chunks:
        m.is_last_microbatch = False

    if len(chunks) > 1:
        if n % pp == 0:
            return _interleaved_schedule(trainer, data, p2p, total)
        return _chunked_schedule(trainer, data, p2p, total)

    model = chunks[0]
    first, last = rank == 0, rank == pp - 1
    warm = min(pp - rank - 1, n)
    inputs: List[Optional[torch.Tensor]] = []
    outputs: List[torch.Tensor] = []

    def fwd(i):
        nonlocal total
        x = None if first else p2p.recv(p2p.prev, _local_rows(data[i], cfg), H)
        out = _forward(trainer, model, data[i], x, n, last)
        if last:
            total += out.detach().float()
        else:
            p2p.send(out, p2p.next)
        inputs.append(x)
        outputs.append(out)

    def bwd(j):
        g = None if last else p2p.recv(p2p.next, outputs[j].shape[0], H, grad=True)
        model.is_last_microbatch = (j == n - 1)
        gi = _backward(outputs[j], g, inputs[j])
        if not first:
            p2p.send(gi, p2p.prev, grad=True)
        inputs[j] = outputs[j] = None

    for i in range(warm):
        fwd(i)
    for k in range(n - warm):
        fwd(warm + k)
        bwd(k)
    for j in range(n - warm, n):
        bwd(j)
    p2p.drain()
    return total


def _chunked_schedule(trainer, data, p2p: _P2P, total: torch.Tensor) -> torch.Tensor:
    """Virtual pipeline: virtual stage ``v = chunk * pp + rank``; data flows v -> v+1."""
    cfg = trainer.config
    pp, rank = ps.get_pipeline_model_parallel_world_size(), ps.get_pipeline_model_parallel_rank()
    n, V, H = len(data), len(trainer.ddp), _pipeline_width(trainer)
    saved = {}
    for c in range(V):
        model = trainer.ddp[c]
        very_first, very_last = (c == 0 and rank == 0), (c == V - 1 and rank == pp - 1)
        for i in range(n):
            x = None if very_first else p2p.recv(p2p.prev, _local_rows(data[i], cfg), H)
            out = _forward(trainer, model, data[i], x, n, very_last)
            if very_last:
                total += out.detach().float()
            else:
                p2p.send(out, p2p.next)
            saved[(c, i)] = (x, out)
        p2p.drain()
    for c in reversed(range(V)):
        model = trainer.ddp[c]
        very_first, very_last = (c == 0 and rank == 0), (c == V - 1 and rank == pp - 1)
        for i in range(n):
            x, out = saved.pop((c, i))
            g = None if very_last else p2p.recv(p2p.next, out.shape[0], H, grad=True)
            model.is_last_microbatch = (i == n - 1)
            gi = _backward(out, g, x)
            if not very_first:
                p2p.send(gi, p2p.prev, grad=True)
        p2p.drain()
    return total


def _interleaved_schedule(trainer, data, p2p: _P2P, total: torch.Tensor) -> torch.Tensor:
    """Interleaved 1F1B over ``V`` model chunks per rank (virtual stage ``v = chunk * pp + rank``).  Step ``k`` of the
    forward (backward) sequence works on chunk ``(k % (pp * V)) // pp`` (mirrored for backward) and micro-batch
    ``(k // (pp * V)) * pp + k % pp``."""
    cfg = trainer.config
    pp, rank = ps.get_pipeline_model_parallel_world_size(), ps.get_pipeline_model_parallel_rank()
    n, V, H = len(data), len(trainer.ddp), _pipeline_width(trainer)
    steps = n * V
    warm = min((pp - rank - 1) * 2 + (V - 1) * pp, steps)
    saved = {}
    done_bwd = [0] * V

    def where(k: int, forward: bool):
        c = (k % (pp * V)) // pp
        if not forward:
            c = V - 1 - c
        return c, (k // (pp * V)) * pp + k % pp

    def fwd(k):
        nonlocal total
        c, i = where(k, True)
        model = trainer.ddp[c]
        very_first, very_last = (c == 0 and rank == 0), (c == V - 1 and rank == pp - 1)
        x = None if very_first else p2p.recv(p2p.prev, _local_rows(data[i], cfg), H)
        out = _forward(trainer, model, data[i], x, n, very_last)
        if very_last:
            total += out.detach().float()
        else:
            p2p.send(out, p2p.next)
        saved[(c, i)] = (x, out)

    def bwd(k):
        c, i = where(k, False)
        model = trainer.ddp[c]
        very_first, very_last = (c == 0 and rank == 0), (c == V - 1 and rank == pp - 1)
        x, out = saved.pop((c, i))
        g = None if very_last else p2p.recv(p2p.next, out.shape[0], H, grad=True)
        done_bwd[c] += 1
        model.is_last_microbatch = (done_bwd[c] == n)     # this chunk's gradients are complete after this backward
        gi = _backward(out, g, x)
        if not very_first:
            p2p.send(gi, p2p.prev, grad=True)

    for k in range(warm):
        fwd(k)
    for k in range(steps - warm):
        fwd(warm + k)
        bwd(k)
    for k in range(steps - warm, steps):
        bwd(k)
    p2p.drain()
    return total
