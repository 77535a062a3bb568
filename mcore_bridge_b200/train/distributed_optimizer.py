"""Data-parallel gradient buffers and the sharded ("distributed") AdamW optimizer.

Layout.  Parameters are regrouped into a few flat buffers keyed by (expert / dense, weight-decay / none):
a bf16 parameter buffer (the model's parameters become views into it) and an fp32 gradient buffer
(``param.main_grad`` views; the weight-gradient GEMMs accumulate straight into it).  Each buffer is cut into
buckets; a bucket is reduce-scattered over the data-parallel group as soon as every gradient in it is
final — on a side stream, overlapping with the rest of backward — and each rank keeps fp32 master weights
and Adam moments only for its 1/dp slice of every bucket.  After the fused Adam kernel has updated the slice
and written the bf16 values, the parameter buffer is all-gathered bucket by bucket.

Dense parameters shard over the ``dp_cp`` group, expert parameters over ``edp``.  Parameters flagged
``sequence_parallel`` (norm weights, router ...) have their gradients summed over the tensor-parallel group
first.  With a data-parallel size of one the collectives vanish and the optimizer still runs the same
fused kernel on the whole buffer.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Iterable, List, Tuple

import torch
import torch.distributed as dist
from torch import nn

from ..ops import _lib
from ..parallel import state as ps
from ..utils.logger import get_logger

logger = get_logger()
_ll, _int, _f = ctypes.c_longlong, ctypes.c_int, ctypes.c_float
ALIGN = 128  # elements; keeps every shard 16-byte aligned for vector access in any dtype


class Bucket:

    def __init__(self, start: int, end: int):
        self.start, self.end = start, end
        self.params: List[nn.Parameter] = []
        self.pending = 0
        self.work = None


class ParamAndGradBuffer:

    def __init__(self, params: List[nn.Parameter], group_name: str, bucket_bytes: int, device, param_dtype,
                 grad_dtype=torch.float32):
        self.group_name = group_name
        self.dp = ps.get_world_size(group_name)
        self.dp_rank = ps.get_rank_in(group_name) if self.dp > 1 else 0
        self.group = ps.get_group(group_name) if self.dp > 1 else None
        # Number of ranks whose losses are averaged into one step.  An expert's gradient already sums the tokens that
        # the ranks of its expert-parallel group sent to it, and is then summed over the expert data-parallel group, so
        # its divisor is the dense data-parallel size as well, not the size of the group it is reduced over.
        self.grad_divisor = max(1, ps.get_world_size('dp_cp'))
        self.params = params
        unit = ALIGN * self.dp
        bucket_elems = max(unit, bucket_bytes // 4 // unit * unit)
        self.buckets: List[Bucket] = []
        self.param_range: Dict[nn.Parameter, Tuple[int, int]] = {}
        offset, bstart = 0, 0
        cur: List[nn.Parameter] = []
        for p in params:
            n = p.numel()
            start = (offset + 7) // 8 * 8
            self.param_range[p] = (start, start + n)
            offset = start + n
            cur.append(p)
            if offset - bstart >= bucket_elems:
                end = (offset + unit - 1) // unit * unit
                b = Bucket(bstart, end)
                b.params = cur
                self.buckets.append(b)
                cur, bstart, offset = [], end, end
        if cur:
            end = (offset + unit - 1) // unit * unit
            b = Bucket(bstart, end)
            b.params = cur
            self.buckets.append(b)
            offset = end
        self.numel = offset
        # With 2..8 ranks of one node the two flat buffers live in peer-mapped memory and the reduce-scatter /
        # all-gather below are in-tree kernels that read the other ranks' buffers over NVLink
        from ..parallel import dp_comm
        self.fused = self.dp > 1 and grad_dtype == torch.float32 and dp_comm.usable(group_name, device)
        if self.fused:
            self.param_ws, self.param_data = dp_comm.allocate(group_name, self.numel, param_dtype)
            self.grad_ws, self.grad_data = dp_comm.allocate(group_name, self.numel, grad_dtype)
        else:
            self.param_data = torch.zeros(self.numel, dtype=param_dtype, device=device)
            self.grad_data = torch.zeros(self.numel, dtype=grad_dtype, device=device)
        self.param_to_bucket: Dict[nn.Parameter, Bucket] = {}
        for b in self.buckets:
            for p in b.params:
                self.param_to_bucket[p] = b
        for p in params:
            s, e = self.param_range[p]
            view = self.param_data[s:e].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad_data[s:e].view(p.shape)

    def shard_range(self, b: Bucket) -> Tuple[int, int]:
        n = (b.end - b.start) // self.dp
        return b.start + self.dp_rank * n, b.start + (self.dp_rank + 1) * n


class DistributedDataParallel(nn.Module):
    """Owns the flat buffers of a model chunk and overlaps gradient reduce-scatter with backward."""

    def __init__(self, module: nn.Module, bucket_mb: float = 256.0, overlap_grad_reduce: bool = True,
                 grad_dtype=torch.float32):
        super().__init__()
        self.module = module
        self.overlap = overlap_grad_reduce
        groups: Dict[Tuple[bool, bool], List[nn.Parameter]] = {}
        seen = set()
        plist = [p for p in module.parameters() if p.requires_grad]
        for p in reversed(plist):  # backward produces gradients roughly in reverse registration order
            if id(p) in seen:
                continue
            seen.add(id(p))
            is_expert = bool(getattr(p, 'is_expert', False))
            decay = p.dim() >= 2 and not getattr(p, 'no_weight_decay', False)
            groups.setdefault((is_expert, decay), []).append(p)
        self.buffers: Dict[Tuple[bool, bool], ParamAndGradBuffer] = {}
        for key, params in groups.items():
            dev, dt = params[0].device, params[0].dtype
            same = [p for p in params if p.dtype == dt]
            assert len(same) == len(params), 'all parameters of a buffer must share a dtype'
            self.buffers[key] = ParamAndGradBuffer(params, 'edp' if key[0] else 'dp_cp', int(bucket_mb * 2**20), dev,
                                                   dt, grad_dtype)
        self.is_last_microbatch = True
        self._comm_stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self._hooks = []
        for buf in self.buffers.values():
            for p in buf.params:
                p.grad_ready_hook = self._make_ready_hook(buf, p)
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_accum_hook(buf, p)))
        self._reset_pending()

    # ------------------------------------------------------------------ hooks
    def _make_accum_hook(self, buf, p):
        def hook(param):
            # The accumulate node also runs for a weight whose backward wrote straight into ``main_grad`` and returned
            # no gradient; that backward has already reported the weight, and a second report would start the bucket's
            # reduction while later gradients are still missing.
            if param.grad is None:
                return
            param.main_grad.add_(param.grad.to(param.main_grad.dtype))
            param.grad = None
            param.grad_ready_hook()
        return hook

    def _make_ready_hook(self, buf: ParamAndGradBuffer, p):
        def ready():
            if not (self.overlap and self.is_last_microbatch and buf.dp > 1):
                return
            b = buf.param_to_bucket[p]
            b.pending -= 1
            if b.pending == 0:
                self._launch_reduce(buf, b)
        return ready

    def _reset_pending(self):
        for buf in self.buffers.values():
            for b in buf.buckets:
                # a parameter used twice in the graph (tied embedding / head) reports twice
                b.pending = sum(int(getattr(p, 'grad_contributions', 1)) for p in b.params)
                b.work = None

    def _needs_tp_reduce(self, b: Bucket) -> bool:
        if ps.get_world_size('tp') > 1 and any(getattr(p, 'sequence_parallel', False) for p in b.params):
            return True
        # copies of a tied embedding on the first and last pipeline stage sum their gradients first
        return ps.get_world_size('embd') > 1 and any(getattr(p, 'shared_embedding', False) for p in b.params)

    def _launch_reduce(self, buf: ParamAndGradBuffer, b: Bucket):
        if buf.dp == 1 or b.work is not None:
            return
        if self._needs_tp_reduce(b):
            return  # reduced in finish_grad_sync after the tensor-parallel all-reduce of flagged grads
        g = buf.grad_data[b.start:b.end]
        s, e = buf.shard_range(b)
        out = buf.grad_data[s:e]
        if g.is_cuda:
            self._comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._comm_stream):
                if buf.fused:
                    from ..parallel import dp_comm
                    dp_comm.reduce_scatter_(buf.grad_ws, buf.grad_data, b.start, b.end)
                    b.work = True       # ordered on the side stream; finish_grad_sync joins the streams
                else:
                    b.work = dist.reduce_scatter_tensor(out, g, group=buf.group, async_op=True)
        else:
            tmp = g.clone()
            dist.all_reduce(tmp, group=buf.group)
            out.copy_(tmp[s - b.start:e - b.start])
            b.work = True

    # ------------------------------------------------------------------ API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def zero_grad_buffer(self):
        for buf in self.buffers.values():
            buf.grad_data.zero_()
        self._reset_pending()

    def _allreduce_sequence_parallel_grads(self):
        if ps.get_world_size('tp') == 1:
            return
        ps_list = [p for buf in self.buffers.values() for p in buf.params if getattr(p, 'sequence_parallel', False)]
        if not ps_list:
            return
        flat = torch.cat([p.main_grad.reshape(-1) for p in ps_list])
        dist.all_reduce(flat, group=ps.get_group('tp'))
        off = 0
        for p in ps_list:
            n = p.numel()
            p.main_grad.copy_(flat[off:off + n].view(p.shape))
            off += n

    def _allreduce_shared_embedding_grads(self):
        """Tied input / output embeddings under pipeline parallelism: the first stage's embedding and the last
        stage's head are two copies of one weight, so their gradients are summed over the two-rank embedding group
        (before the data-parallel reduction, while every rank still holds full gradients)."""
        if ps.get_world_size('embd') == 1:
            return
        for buf in self.buffers.values():
            for p in buf.params:
                if getattr(p, 'shared_embedding', False):
                    dist.all_reduce(p.main_grad, group=ps.get_group('embd'))

    def finish_grad_sync(self):
        """Blocks until every bucket's gradient shard is reduced (launching the ones not started yet)."""
        self._allreduce_sequence_parallel_grads()
        self._allreduce_shared_embedding_grads()
        for buf in self.buffers.values():
            if buf.dp == 1:
                continue
            for b in buf.buckets:
                if b.work is None:
                    g = buf.grad_data[b.start:b.end]
                    s, e = buf.shard_range(b)
                    if g.is_cuda and buf.fused:
                        # same side stream as the overlapped buckets: the kernels of one buffer never run concurrently
                        from ..parallel import dp_comm
                        self._comm_stream.wait_stream(torch.cuda.current_stream())
                        with torch.cuda.stream(self._comm_stream):
                            dp_comm.reduce_scatter_(buf.grad_ws, buf.grad_data, b.start, b.end)
                    elif g.is_cuda:
                        dist.reduce_scatter_tensor(buf.grad_data[s:e], g, group=buf.group)
                    else:
                        tmp = g.clone()
                        dist.all_reduce(tmp, group=buf.group)
                        buf.grad_data[s:e].copy_(tmp[s - b.start:e - b.start])
                elif b.work is not True:
                    b.work.wait()
        if self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, *a, **k):
        return self.module.load_state_dict(*a, **k)


_WITH_PENDING_GATHERS = None      # weak set of optimizers created with overlap_param_gather


def finish_all_param_gathers() -> None:
    """Waits for the overlapped parameter all-gathers of every live optimizer; the checkpoint bridge calls it before
    it reads parameters.  A no-op unless an optimizer was built with ``overlap_param_gather``."""
    if _WITH_PENDING_GATHERS:
        for opt in list(_WITH_PENDING_GATHERS):
            opt.finish_param_gather()


class DistributedOptimizer:
    """AdamW on the rank's slice of every bucket; fp32 master weights + moments are allocated only for it."""

    def __init__(self, ddp_models: Iterable[DistributedDataParallel], lr: float = 1e-4, betas=(0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.1, clip_grad: float = 1.0,
                 overlap_param_gather: bool = False):
        self.models = list(ddp_models)
        self.lr, self.betas, self.eps, self.weight_decay, self.clip_grad = lr, betas, eps, weight_decay, clip_grad
        self.step_count = 0
        self.shards = []  # (buf, bucket, decay, main, m, v)
        for model in self.models:
            for (is_expert, decay), buf in model.buffers.items():
                for b in buf.buckets:
                    s, e = buf.shard_range(b)
                    main = buf.param_data[s:e].float().clone()
                    self.shards.append((buf, b, decay, main, torch.zeros_like(main), torch.zeros_like(main)))
        dev = self.shards[0][3].device if self.shards else torch.device('cpu')
        self.device = dev
        self._scalars = {True: torch.zeros(8, dtype=torch.float32, device=dev),
                         False: torch.zeros(8, dtype=torch.float32, device=dev)}
        # [0] sum of squared gradients; [1] number of ranks whose kernel status word is raised (both all-reduced)
        self._sq = torch.zeros(2, dtype=torch.float32, device=dev)
        self._sq_scratch = None
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)   # != 0: this step's update is not applied
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_norm = self._norm
        self.grad_scale = 1.0
        # overlap_param_gather: the all-gather of the updated parameters is issued bucket by bucket in the order the
        # next forward pass needs them (on a side stream on a GPU, as asynchronous collectives elsewhere) and every
        # transformer layer waits only for its own buckets
        self.overlap_param_gather = bool(overlap_param_gather)
        self._pending: Dict[int, tuple] = {}
        self._gather_order: List[Tuple[ParamAndGradBuffer, Bucket]] = []
        self._ag_stream = None
        if self.overlap_param_gather:
            self._install_gather_hooks()
            global _WITH_PENDING_GATHERS
            if _WITH_PENDING_GATHERS is None:
                import weakref
                _WITH_PENDING_GATHERS = weakref.WeakSet()
            _WITH_PENDING_GATHERS.add(self)

    def zero_grad(self):
        for m in self.models:
            m.zero_grad_buffer()

    def _use_cuda(self):
        return self.device.type == 'cuda' and _lib.available()

    def _grad_norm(self):
        """Global L2 norm over every distinct gradient element (dp-sharded, tp-sharded, pp-sharded)."""
        self._sq.zero_()
        tp_rank0 = ps.get_rank_in('tp') == 0 if ps.get_world_size('tp') > 1 else True
        # A shard holds the *sum* of the data-parallel ranks' gradients; the averaging (and any loss scale) is folded
        # into the optimizer kernel's gradient scale.  The norm is that of the gradient the update uses, so every
        # buffer's sum of squares is scaled accordingly (buffers can have different data-parallel sizes: dense vs
        # expert).
        part = torch.zeros(1, dtype=torch.float32, device=self._sq.device)
        cur = None
        tied_copy = ps.get_world_size('embd') > 1 and not ps.is_pipeline_first_stage()

        def flush():
            if cur is not None:
                self._sq[0:1].add_(part * (self.grad_scale / cur.grad_divisor) ** 2)
                part.zero_()

        for buf, b, decay, main, m, v in self.shards:
            if buf is not cur:
                flush()
                cur = buf
            s, e = buf.shard_range(b)
            g = buf.grad_data[s:e]
            # replicated (non tensor-parallel) parameters are counted once per TP group
            if not tp_rank0 and ps.get_world_size('tp') > 1:
                dup = self._replicated_mask(buf, b, s, e)
                if dup is not None:
                    g = g * dup
            # a tied embedding lives on the first and on the last pipeline stage (both hold the summed gradient):
            # the first stage's copy is the one that counts
            if tied_copy:
                dup = self._replicated_mask(buf, b, s, e, lambda p: getattr(p, 'shared_embedding', False))
                if dup is not None:
                    g = g * dup
            if self._use_cuda() and g.dtype == torch.float32:
                if self._sq_scratch is None:     # per-CTA partials + ticket: fixed summation order
                    self._sq_scratch = torch.zeros(1025, dtype=torch.float32, device=g.device)
                _lib.check_rc(_lib.lib().mcb_sqnorm_accum(_lib.ptr(g), _ll(g.numel()), _lib.ptr(part),
                                                          _lib.ptr(self._sq_scratch), _lib.stream_ptr()),
                              'mcb_sqnorm_accum')
            else:
                part += g.float().pow(2).sum()
        flush()
        if self._use_cuda():
            # a raised status word (a bounded wait that gave up, an overflowing MoE receive buffer) on any rank makes
            # every rank skip the update: the flag rides along with the norm's all-reduce, no host round trip
            self._sq[1:2].copy_((_lib.status_word(self.device)[0:1] != 0).float())
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self._sq)  # shards are disjoint across all ranks except the masked replicas
        self._skip.copy_((self._sq[1:2] > 0).int())
        if self._use_cuda():
            _lib.check_rc(_lib.lib().mcb_clip_coef(_lib.ptr(self._sq), _f(float(self.clip_grad or 0.0)),
                                                   _lib.ptr(self._coef), _lib.ptr(self._norm), _lib.stream_ptr()),
                          'mcb_clip_coef')
        else:
            self._norm.copy_(self._sq[0:1].sqrt())
            if self.clip_grad and self.clip_grad > 0:
                self._coef.copy_(torch.clamp(self.clip_grad / (self._norm + 1e-6), max=1.0))
            else:
                self._coef.fill_(1.0)

    def _replicated_mask(self, buf, b, s, e, duplicate=None):
        """0 over the part of the shard ``[s, e)`` that belongs to parameters another rank already counts (by default
        the parameters replicated over the tensor-parallel group), 1 elsewhere; ``None`` when nothing is masked."""
        if duplicate is None:
            def duplicate(p):
                return not (getattr(p, 'tensor_model_parallel', False) or getattr(p, 'is_expert', False))
        mask = None
        for p in b.params:
            if not duplicate(p):
                continue
            ps_, pe = buf.param_range[p]
            lo, hi = max(ps_, s), min(pe, e)
            if lo < hi:
                if mask is None:
                    mask = torch.ones(e - s, dtype=torch.float32, device=buf.grad_data.device)
                mask[lo - s:hi - s] = 0
        return mask

    @torch.no_grad()
    def step(self):
        for m in self.models:
            m.finish_grad_sync()
        self.step_count += 1
        t = self.step_count
        b1, b2 = self.betas
        self._grad_norm()
        for decay in (True, False):
            # data-parallel averaging is folded into the gradient scale
            self._scalars[decay].copy_(torch.tensor(
                [self.lr, b1, b2, self.eps, self.weight_decay if decay else 0.0, 1 - b1**t, 1 - b2**t, self.grad_scale],
                dtype=torch.float32), non_blocking=True)
        for buf, b, decay, main, m, v in self.shards:
            s, e = buf.shard_range(b)
            g = buf.grad_data[s:e]
            pshard = buf.param_data[s:e]
            scale_dp = 1.0 / buf.grad_divisor
            if self._use_cuda() and g.dtype == torch.float32 and pshard.dtype in (torch.bfloat16, torch.float32):
                sc = self._scalars[decay]
                if scale_dp != 1.0:
                    sc = sc.clone()
                    sc[7] *= scale_dp
                rc = _lib.lib().mcb_adam_step(_lib.ptr(g), _lib.ptr(main), _lib.ptr(m), _lib.ptr(v), _lib.ptr(pshard),
                                              _int(int(pshard.dtype == torch.bfloat16)), _ll(main.numel()),
                                              _lib.ptr(sc), _lib.ptr(self._coef), _lib.ptr(self._skip),
                                              _lib.stream_ptr())
                _lib.check_rc(rc, 'mcb_adam_step')
            else:
                gf = g.float() * (self.grad_scale * scale_dp) * self._coef
                m.mul_(b1).add_(gf, alpha=1 - b1)
                v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
                denom = (v / (1 - b2**t)).sqrt_().add_(self.eps)
                main.mul_(1 - self.lr * (self.weight_decay if decay else 0.0))
                main.addcdiv_(m / (1 - b1**t), denom, value=-self.lr)
                pshard.copy_(main.to(pshard.dtype))
        # parameter all-gather, bucket by bucket (in place: every rank's slice sits at its final position)
        if self.overlap_param_gather:
            self._start_param_gather()
            return self._norm
        for buf, b, *_ in self.shards:
            if buf.dp > 1:
                self._gather_bucket(buf, b)
        return self._norm

    @staticmethod
    def _gather_bucket(buf: ParamAndGradBuffer, b: Bucket, async_op: bool = False):
        full = buf.param_data[b.start:b.end]
        s, e = buf.shard_range(b)
        if full.is_cuda and buf.fused:
            from ..parallel import dp_comm
            dp_comm.all_gather_(buf.param_ws, buf.param_data, b.start, b.end)
        elif full.is_cuda:
            dist.all_gather_into_tensor(full, buf.param_data[s:e], group=buf.group)
        else:
            parts = [torch.empty_like(buf.param_data[s:e]) for _ in range(buf.dp)]
            work = dist.all_gather(parts, buf.param_data[s:e].clone(), group=buf.group, async_op=async_op)
            if async_op:
                return work, parts, full
            full.copy_(torch.cat(parts))
        return None

    # ------------------------------------------------------------------ overlapped parameter all-gather
    def _install_gather_hooks(self):
        """Forward pre-hooks: the model waits for the buckets that hold parameters outside the transformer layers
        (embedding, head, final norm, towers), each transformer layer for the buckets that hold its own.  The issue
        order follows the same sequence, so on a GPU a layer's wait never covers a later layer's bucket."""
        from ..models.transformer_layer import TransformerLayer
        for model in self.models:
            p2b = {}
            for buf in model.buffers.values():
                if buf.dp > 1:
                    for p, b in buf.param_to_bucket.items():
                        p2b[p] = (buf, b)
            layers = [m for m in model.module.modules() if isinstance(m, TransformerLayer)]
            in_layer = set()
            per_layer = []
            for lay in layers:
                own = []
                for p in lay.parameters():
                    in_layer.add(p)
                    if p in p2b and p2b[p] not in own:
                        own.append(p2b[p])
                per_layer.append(own)
            root = []
            for p, bb in p2b.items():
                if p not in in_layer and bb not in root:
                    root.append(bb)
            for bb in root + [bb for own in per_layer for bb in own]:
                if bb not in self._gather_order:
                    self._gather_order.append(bb)

            def make_hook(buckets):
                ids = [id(b) for _, b in buckets]

                def hook(module, args):
                    if self._pending:
                        self._wait_buckets(ids)
                return hook

            model.module.register_forward_pre_hook(make_hook(root))
            for lay, own in zip(layers, per_layer):
                lay.register_forward_pre_hook(make_hook(own))

    def _start_param_gather(self):
        self.finish_param_gather()
        on_gpu = self.device.type == 'cuda'
        if on_gpu:
            if self._ag_stream is None:
                self._ag_stream = torch.cuda.Stream()
            self._ag_stream.wait_stream(torch.cuda.current_stream())
        for buf, b in self._gather_order:
            if on_gpu:
                with torch.cuda.stream(self._ag_stream):
                    self._gather_bucket(buf, b)
                    ev = torch.cuda.Event()
                    ev.record(self._ag_stream)
                self._pending[id(b)] = ('event', ev)
            else:
                self._pending[id(b)] = ('work',) + self._gather_bucket(buf, b, async_op=True)

    def _wait_buckets(self, ids):
        for i in ids:
            item = self._pending.pop(i, None)
            if item is None:
                continue
            if item[0] == 'event':
                torch.cuda.current_stream().wait_event(item[1])
            else:
                _, work, parts, full = item
                work.wait()
                with torch.no_grad():
                    full.copy_(torch.cat(parts))

    def finish_param_gather(self):
        """Waits for every parameter all-gather still in flight.  Anything that reads parameters without running the
        model's forward pass (a hand-written loop over ``model.parameters()``) calls this first; ``state_dict``, the
        next ``step`` and the checkpoint bridge's export do it themselves."""
        if self._pending:
            self._wait_buckets(list(self._pending))

    def undo_skipped_step(self):
        """After a step whose update the device-side flag suppressed: take the step count back so the bias corrections
        of the repeated step are the right ones."""
        self.step_count -= 1

    @property
    def skip_flag(self) -> torch.Tensor:
        """int32[1] on the device: non-zero when the last ``step()`` left parameters and moments untouched."""
        return self._skip

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        self.finish_param_gather()
        return {
            'step': self.step_count,
            'shards': [{'main': main, 'exp_avg': m, 'exp_avg_sq': v} for (_, _, _, main, m, v) in self.shards],
            'hyper': {'lr': self.lr, 'betas': self.betas, 'eps': self.eps, 'weight_decay': self.weight_decay},
        }

    def load_state_dict(self, sd: dict):
        self.step_count = int(sd['step'])
        assert len(sd['shards']) == len(self.shards), 'optimizer shard layout changed'
        for (_, _, _, main, m, v), s in zip(self.shards, sd['shards']):
            main.copy_(s['main'])
            m.copy_(s['exp_avg'])
            v.copy_(s['exp_avg_sq'])
