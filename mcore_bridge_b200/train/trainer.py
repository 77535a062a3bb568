"""Training entry point: build model + optimizer, run steps.  ``Trainer.train_step`` is the call a user makes.

A step = ``num_microbatches`` forward/backward passes (activation recompute per config) with gradient
accumulation in the fp32 buffers, then gradient reduce-scatter, clipping, fused AdamW on the local shards
and parameter all-gather.  Inputs arrive as host tensors (pinned when possible) and are copied to the device
inside the step; the loss comes back to the host at the end of the step.  Pipeline parallel runs go through
``train/schedules.py``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

from ..layers.context import PackedSeqParams
from ..layers.moe import get_moe_aux_losses
from ..models.register import get_mcore_model
from ..ops.moe import MoEAuxLossAutoScaler
from ..parallel import state as ps
from ..utils.logger import get_logger
from ..utils.megatron_utils import split_cp_inputs
from ..utils.profiling import _NO_RANGE, DeviceTimers, nvtx_range
from ..utils.torch_utils import attach_host_list
from .distributed_optimizer import DistributedDataParallel, DistributedOptimizer

logger = get_logger()


@dataclass
class TrainConfig:
    lr: float = 1e-4
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.1
    clip_grad: float = 1.0
    bucket_mb: float = 256.0
    overlap_grad_reduce: bool = True
    overlap_param_gather: bool = False     # parameter all-gather of step N overlaps the forward pass of step N + 1
    init_seed: Optional[int] = 1234
    init_std: float = 0.02
    device_timers: bool = False            # CUDA-event time of forward+backward and of the optimizer in last_metrics
    heartbeat_dir: Optional[str] = None    # when set, every step touches this rank's heartbeat file (train/health.py)
    heartbeat_timeout_s: float = 60.0


_BATCH_KEYS = frozenset({'input_ids', 'labels', 'position_ids', 'attention_mask', 'loss_mask', 'cu_seqlens',
                         'max_seqlen'})


def model_extras(d: Dict) -> Dict:
    """What a micro-batch holds beyond the text fields (``pixel_values``, ``image_grid_thw``, ``input_features`` ...):
    passed to the model as keyword arguments, for the multimodal wrappers."""
    return {k: v for k, v in d.items() if k not in _BATCH_KEYS}


@torch.no_grad()
def init_weights(model: torch.nn.Module, std: float = 0.02, seed: Optional[int] = None):
    """Random init: N(0, std) for matrices (tensor-parallel shards draw from the TP stream, replicated tensors
    from the shared stream), norms at their identity value, biases zero."""
    from ..parallel.random import get_rng_tracker, model_parallel_manual_seed
    if seed is not None:
        model_parallel_manual_seed(seed)
    tracker = get_rng_tracker()
    for name, p in model.named_parameters():
        is_norm = ('layernorm' in name or 'layer_norm' in name or name.endswith('norm.weight') or
                   'q_norm' in name or 'k_norm' in name)
        if p.dim() < 2 and (is_norm or name.endswith('bias')):
            if is_norm and name.endswith('weight'):
                zero_centered = (getattr(model, 'config', None) is not None
                                 and model.config.layernorm_zero_centered_gamma)
                p.fill_(0.0 if zero_centered else 1.0)
            else:
                p.zero_()
            continue
        if p.dim() < 2:
            continue  # family-specific 1-D parameters (A_log, dt_bias ...) keep their constructor values
        stream = 'expert-parallel-rng' if getattr(p, 'is_expert', False) else (
            'model-parallel-rng' if getattr(p, 'tensor_model_parallel', False) else None)
        if stream is not None and stream in tracker.states:
            with tracker.fork(stream):
                p.normal_(0.0, std)
        else:
            p.normal_(0.0, std)


def sync_shared_embeddings(models) -> None:
    """Makes the last pipeline stage's copy of a tied embedding equal to the first stage's (after random init; a
    checkpoint load fills both from the same tensor anyway)."""
    if ps.get_world_size('embd') == 1:
        return
    src = ps.get_group_ranks('embd')[0]
    for m in models:
        for p in m.parameters():
            if getattr(p, 'shared_embedding', False):
                dist.broadcast(p.data, src=src, group=ps.get_group('embd'))


class Trainer:

    def __init__(self, config, train_config: Optional[TrainConfig] = None, models: Optional[List] = None):
        self.config = config
        self.tc = train_config or TrainConfig()
        self.models = models if models is not None else get_mcore_model(config)
        if models is None and self.tc.init_seed is not None:
            for i, m in enumerate(self.models):
                init_weights(m, self.tc.init_std, self.tc.init_seed + i)
        sync_shared_embeddings(self.models)
        self.ddp = [DistributedDataParallel(m, self.tc.bucket_mb, self.tc.overlap_grad_reduce) for m in self.models]
        self.optimizer = DistributedOptimizer(self.ddp, self.tc.lr, self.tc.betas, self.tc.eps, self.tc.weight_decay,
                                              self.tc.clip_grad, overlap_param_gather=self.tc.overlap_param_gather)
        self.device = next(self.models[0].parameters()).device
        self.timers = DeviceTimers() if self.tc.device_timers else None
        # MCB200_CHECK_COLLECTIVES=1: every collective is compared across its group on the host before it is launched
        self._collective_checker = None
        from ..parallel import collective_check
        if collective_check.enabled_by_env() and dist.is_available() and dist.is_initialized() \
                and dist.get_world_size() > 1:
            self._collective_checker = collective_check.CollectiveOrderChecker().install()
        self._copy_stream = torch.cuda.Stream() if self.device.type == 'cuda' else None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.last_metrics: Dict[str, float] = {}
        self._hb = None

    # ------------------------------------------------------------------ data movement
    def _to_device(self, mb: Dict) -> Dict:
        out = {}
        for k, v in mb.items():
            if isinstance(v, torch.Tensor):
                self.h2d_bytes += v.numel() * v.element_size() if v.device.type == 'cpu' else 0
                out[k] = v.to(self.device, non_blocking=True)
                if k == 'cu_seqlens':      # the layers that walk the boundaries on the host read them from here
                    attach_host_list(out[k], v)
            else:
                out[k] = v
        return out

    def _prepare(self, mb: Dict) -> Dict:
        """Device copy + context-parallel selection of this rank's zig-zag chunks."""
        d = self._to_device(mb)
        cp = ps.get_world_size('cp')
        if cp > 1:
            cu = d.get('cu_seqlens')
            for k in ('input_ids', 'labels', 'position_ids', 'loss_mask'):
                if d.get(k) is not None:
                    d[k] = split_cp_inputs(d[k], cu, -1)
        return d

    # ------------------------------------------------------------------ one micro-batch
    def forward_backward_microbatch(self, d: Dict, num_microbatches: int) -> torch.Tensor:
        model = self.ddp[0]
        psp = None
        if d.get('cu_seqlens') is not None:
            psp = PackedSeqParams(cu_seqlens_q=d['cu_seqlens'], cu_seqlens_kv=d['cu_seqlens'],
                                  max_seqlen_q=d.get('max_seqlen'), max_seqlen_kv=d.get('max_seqlen'))
        loss_tok = model(input_ids=d['input_ids'], position_ids=d.get('position_ids'),
                         attention_mask=d.get('attention_mask'), labels=d['labels'], packed_seq_params=psp,
                         loss_mask=d.get('loss_mask'), **model_extras(d))
        mask = d.get('loss_mask')
        if mask is None:
            mask = torch.ones_like(loss_tok)
        ntok = mask.sum()
        cpn = ps.get_world_size('cp')
        if cpn > 1:
            ntok = ntok.clone()
            dist.all_reduce(ntok, group=ps.get_group('cp'))
        # Under context parallelism every rank holds part of each sequence and the sum above is normalised by the
        # micro-batch's token count, i.e. it is this rank's *share* of the micro-batch loss.  Gradients are averaged
        # over the dp x cp group, so the share is scaled by cp: the average over the cp ranks is then the micro-batch
        # gradient.  The load-balancing loss is a share in the same sense; the MTP loss is a local mean and is not.
        loss = (loss_tok * mask).sum() / ntok.clamp(min=1.0) * (float(cpn) / num_microbatches)
        MoEAuxLossAutoScaler.set_loss_scale(float(cpn) / num_microbatches)
        from ..layers.mtp import MTPLossAutoScaler
        MTPLossAutoScaler.set_loss_scale(1.0 / num_microbatches)
        loss.backward()
        return loss.detach()

    # ------------------------------------------------------------------ the public step
    def _forward_backward(self, mbs: List[Dict]) -> torch.Tensor:
        n = len(mbs)
        if ps.get_world_size('pp') > 1:
            from .schedules import forward_backward_pipelining
            total = forward_backward_pipelining(self, mbs)
            # only the last stage computed the loss (the others hold zero): give every stage the value
            dist.all_reduce(total, group=ps.get_group('pp'))
            return total
        self.optimizer.zero_grad()
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        nxt = self._prepare(mbs[0])
        for i in range(n):
            cur = nxt
            for m in self.ddp:
                m.is_last_microbatch = (i == n - 1)
            if i + 1 < n:
                nxt = self._prepare(mbs[i + 1])  # async H2D of the next micro-batch overlaps this one's compute
            total += self.forward_backward_microbatch(cur, n)
        return total

    def train_step(self, microbatches: Iterable[Dict]) -> float:
        """Runs one optimizer step over the given host micro-batches and returns the mean loss (host float).

        A kernel that reported a problem during the step (status word raised on any rank) makes the optimizer leave
        the parameters untouched, on the device and without a host round trip; the host learns of it with the loss.
        An overflowing MoE receive buffer is then handled here: the buffers grow and the step is repeated.  Any other
        status raises :class:`KernelError` with the weights still those of the previous step."""
        mbs = list(microbatches)
        if self.tc.heartbeat_dir:
            # between steps, nothing of this rank in flight: publish liveness and learn of ranks that stopped, on the
            # host, before the next launch could wait for them
            hb = self._heartbeat()
            hb.beat(self.optimizer.step_count)
            dead = hb.dead_ranks(missing_is_dead=False)
            if dead:
                from .health import RankFailure
                hb.beat(self.optimizer.step_count, status='peer-failure')
                raise RankFailure(dead)
        for attempt in range(4):
            with nvtx_range('forward_backward'), self._timed('forward_backward'):
                total = self._forward_backward(mbs)
            with nvtx_range('optimizer'), self._timed('optimizer'):
                grad_norm = self.optimizer.step()
            # every rank holds cp x its share of its micro-batches' loss: the mean over the dp x cp group is the step's
            # loss
            if ps.get_world_size('dp_cp') > 1:
                dist.all_reduce(total, group=ps.get_group('dp_cp'))
                total = total / ps.get_world_size('dp_cp')
            out = torch.stack([total.float(), grad_norm.float().reshape(()),
                               self.optimizer.skip_flag.float().reshape(())])
            host = out.cpu()                       # the step's device->host read
            self.d2h_bytes += out.numel() * out.element_size()
            if float(host[2]) == 0.0:
                break
            # the update was suppressed on every rank
            self.optimizer.undo_skipped_step()
            from ..ops import _lib
            code = int(_lib.status_word(self.device)[0].item())
            codes = torch.tensor([code], device=self.device)
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                dist.all_reduce(codes, op=dist.ReduceOp.MAX)          # ST_MOE_OVERFLOW is the largest code
            if int(codes.item()) != _lib.ST_MOE_OVERFLOW or attempt == 3:
                _lib.check_status(self.device)     # raises on the rank(s) that hold the status
                raise _lib.KernelError('another rank reported a kernel status; this step was not applied')
            from ..layers import moe_fused
            _lib.status_word(self.device)[0] = 0
            factor = moe_fused.grow_capacity()
            logger.warning(f'MoE receive buffer overflowed; capacity factor raised to {factor}, repeating the step')
        self._after_step()
        self.last_metrics = {'loss': float(host[0]), 'grad_norm': float(host[1])}
        if self.timers is not None:             # device time of the two phases of this step (CUDA events)
            for name, rec in self.timers.summary().items():
                self.last_metrics[f'{name}_ms'] = rec['total_ms']
        from ..layers.mtp import get_mtp_losses
        for k, (sm, c) in list(get_mtp_losses().items()):
            self.last_metrics[f'mtp_{k + 1}_loss'] = float(sm) / max(c, 1)
        get_mtp_losses().clear()
        aux = get_moe_aux_losses()
        for k, (s, c) in list(aux.items()):
            self.last_metrics[k] = float(s) / max(c, 1)
        aux.clear()
        return self.last_metrics['loss']

    def _timed(self, name: str):
        return self.timers.time(name) if self.timers is not None else _NO_RANGE

    def _heartbeat(self):
        if self._hb is None:
            from .health import HeartbeatMonitor
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
            world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
            self._hb = HeartbeatMonitor(self.tc.heartbeat_dir, rank, world, self.tc.heartbeat_timeout_s)
        return self._hb

    def _after_step(self):
        if self.config.moe_router_enable_expert_bias:
            from ..layers.moe import TopKRouter
            group = ps.get_group('tp_dp_cp') if ps.get_world_size('tp_dp_cp') > 1 else None
            for m in self.models:
                for mod in m.modules():
                    if isinstance(mod, TopKRouter):
                        mod.update_expert_bias(group)
