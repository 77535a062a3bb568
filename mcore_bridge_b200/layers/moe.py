"""Mixture-of-experts layer: router, token dispatcher, grouped experts, shared expert.

Dispatch is "alltoall" (the reference pins ``moe_token_dispatcher_type='alltoall'`` and
``moe_grouped_gemm=True``, ``src/mcore_bridge/config/model_config.py:233-234``): every rank routes its own
tokens, copies travel to the rank owning the expert, experts run as one grouped GEMM over an
expert-sorted buffer, results travel back and are summed per token.

Module / parameter names (``router.weight``, ``router.expert_bias``, ``experts.linear_fc1``,
``shared_experts.gate_weight`` ...) match what the weight bridge addresses.  Expert weights are stored
stacked, ``[E_local, out, in]``, the layout the grouped tcgen05 GEMM consumes; ``weight{i}`` resolves to
a view of expert ``i``.
"""
from __future__ import annotations

import re
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from ..ops import gemm
from ..ops import moe as moe_ops
from ..ops.activation import glu
from ..ops.linear import linear
from ..parallel import mappings as M
from ..parallel import state as ps
from .linear import ColumnParallelLinear, RowParallelLinear, _set_tp_attrs
from .norm import mark_sequence_parallel

_AUX_TRACKER = {}


def get_moe_aux_losses() -> dict:
    """Per-step tracker ``{name: (sum, count)}`` the trainer logs and clears."""
    return _AUX_TRACKER


def _micro_batch_tokens(cfg, ntok_local, ntok_group, group: str):
    """Tokens of the micro-batch this rank holds a slice of.  Under sequence / context parallelism every rank of the
    ``tp_cp`` group sees part of the same micro-batch, and the load-balancing term is linear in the mean probability
    ``P_e``: each rank contributes ``sum of its scores / tokens of the whole micro-batch``, so that the ranks' terms add
    up to the loss of the micro-batch (and each rank's gradient is exactly its share of it)."""
    if group == 'tp_cp':
        return ntok_group
    parts = ps.get_world_size('tp_cp') if (cfg.sequence_parallel or cfg.context_parallel_size > 1) else 1
    return ntok_local * parts


def _track(name: str, value: torch.Tensor):
    s, c = _AUX_TRACKER.get(name, (0.0, 0))
    _AUX_TRACKER[name] = (s + value.detach().float(), c + 1)


def _gate_on_engine(x: torch.Tensor, w: torch.Tensor) -> bool:
    from ..ops import _lib
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[0] % 8 == 0
            and w.shape[1] % 8 == 0 and _lib.available())


class _RouterGateFn(torch.autograd.Function):
    """Router logits ``x @ w^T`` on the tensor-core GEMM.  bf16 operands with fp32 accumulation give the products and
    sums of the fp32 GEMM the router's ``moe_router_dtype='fp32'`` asks for (a bf16 value is exact in fp32).  The
    fp32 logit gradient enters the backward GEMMs as two bf16 terms (value rounded to bf16 + the rounding error), which
    keeps 16 mantissa bits; both terms ride in one GEMM by doubling the contraction dimension."""

    @staticmethod
    def forward(ctx, x, w, out_dtype):
        from ..ops import gemm
        ctx.save_for_backward(x, w)
        return gemm.mm_nt(x, w, out_dtype=out_dtype)

    @staticmethod
    def backward(ctx, dl):
        from ..ops import gemm
        x, w = ctx.saved_tensors
        E = w.shape[0]
        if dl.dtype == torch.float32:
            hi = dl.to(torch.bfloat16)
            d2 = torch.cat([hi, (dl - hi.float()).to(torch.bfloat16)], dim=1)      # [T, 2E]
            w2 = torch.cat([w, w], dim=0)                                          # [2E, H]
        else:
            d2, w2 = dl.contiguous(), w
        dx = gemm.mm_nn(d2, w2) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = gemm.mm_tn(d2, x, out_dtype=torch.float32)                         # [2E or E, H]
            if dw.shape[0] != E:
                dw = dw[:E] + dw[E:]
            dw = dw.to(w.dtype)
        return dx, dw, None


class TopKRouter(nn.Module):
    """Gate ``[E, H]`` in fp32 math + top-k selection + load-balancing losses + expert-bias bookkeeping.

    The expert-bias token count ignores padded tokens and is only updated while gradients are enabled, so
    evaluation and activation recomputation do not double count (reference
    ``src/mcore_bridge/model/modules/topk_router.py:7-21``).
    """

    def __init__(self, config, is_hash_layer: bool = False):
        super().__init__()
        self.config = config
        self.num_experts = config.num_moe_experts
        self.topk = config.moe_router_topk
        self.weight = nn.Parameter(torch.empty(self.num_experts, config.hidden_size, dtype=config.params_dtype))
        _set_tp_attrs(self.weight, False, -1)
        mark_sequence_parallel(self.weight, config)
        if config.add_bias_linear:          # GPT-OSS: biased gate
            self.bias = nn.Parameter(torch.zeros(self.num_experts, dtype=config.params_dtype))
            _set_tp_attrs(self.bias, False, -1)
            mark_sequence_parallel(self.bias, config)
        else:
            self.register_parameter('bias', None)
        # hash-routed layers (the first ``moe_n_hash_layers`` MoE layers of DeepSeek-V4): the experts of a token are a
        # fixed function of its id, read from the table ``tid2eid``; the gate still provides the mixing weights
        self.is_hash_layer = bool(is_hash_layer)
        if self.is_hash_layer:
            self.register_buffer('tid2eid', torch.zeros(config.padded_vocab_size, self.topk, dtype=torch.int64))
        self.enable_expert_bias = bool(config.moe_router_enable_expert_bias)
        if self.enable_expert_bias:
            self.register_buffer('expert_bias', torch.zeros(self.num_experts, dtype=torch.float32))
            self.register_buffer('local_tokens_per_expert', torch.zeros(self.num_experts, dtype=torch.float32),
                                 persistent=False)
        else:
            self.expert_bias = None

    def gating(self, x: torch.Tensor) -> torch.Tensor:
        dt = {None: x.dtype, 'fp32': torch.float32, 'fp64': torch.float64}[self.config.moe_router_dtype]
        if dt != torch.float64 and x.dim() == 2 and _gate_on_engine(x, self.weight):
            logits = _RouterGateFn.apply(x, self.weight, dt)
            return logits if self.bias is None else logits + self.bias.to(dt)
        return torch.nn.functional.linear(x.to(dt), self.weight.to(dt), None if self.bias is None else self.bias.to(dt))

    def _apply_expert_bias(self, indices: torch.Tensor, padding_mask: Optional[torch.Tensor]):
        if self.enable_expert_bias and torch.is_grad_enabled():
            with torch.no_grad():
                valid = None if padding_mask is None else ~padding_mask.reshape(-1)
                self.local_tokens_per_expert += moe_ops.tokens_per_expert(indices, self.num_experts, valid)

    @torch.no_grad()
    def update_expert_bias(self, group=None):
        """Aux-loss-free balancing: ``bias += rate * sign(mean_load - load)`` from the accumulated counts."""
        if not self.enable_expert_bias:
            return
        load = self.local_tokens_per_expert.clone()
        if group is not None:
            dist.all_reduce(load, group=group)
        self.expert_bias += self.config.moe_router_bias_update_rate * torch.sign(load.mean() - load)
        self.local_tokens_per_expert.zero_()

    def _hash_route(self, logits: torch.Tensor, input_ids: torch.Tensor):
        """Experts from the id table, weights from the gate's scores of those experts (normalised over the ``k``
        experts unless the scores are pre-softmax probabilities, then scaled like the learned routing)."""
        cfg = self.config
        if input_ids is None:
            raise ValueError('hash-routed MoE layers need the token ids (ForwardContext.input_ids)')
        ids = input_ids.reshape(-1)
        tp = ps.get_world_size('tp')
        if ids.numel() == logits.shape[0] * tp and cfg.sequence_parallel and tp > 1:
            ids = ids.chunk(tp)[ps.get_rank_in('tp')]         # sequence parallelism: this rank's slice of the tokens
        if ids.numel() != logits.shape[0]:
            raise ValueError(f'hash routing: {ids.numel()} token ids for {logits.shape[0]} tokens (under sequence '
                             'parallelism pass the ids of this rank\'s tokens)')
        idx = self.tid2eid[ids.clamp(min=0)]
        scores = torch.sigmoid(logits.float()) if cfg.moe_router_score_function == 'sigmoid' else \
            torch.softmax(logits.float(), dim=-1)
        probs = scores.gather(1, idx)
        if self.topk > 1 and cfg.moe_router_score_function == 'sigmoid':
            probs = probs / probs.sum(-1, keepdim=True).clamp_min(1e-20)
        if cfg.moe_router_topk_scaling_factor:
            probs = probs * cfg.moe_router_topk_scaling_factor
        return probs.to(logits.dtype), idx, scores

    def forward(self, x: torch.Tensor, padding_mask: Optional[torch.Tensor] = None, seg_ids=None, num_seqs=None,
                input_ids: Optional[torch.Tensor] = None):
        cfg = self.config
        logits = self.gating(x)
        if self.is_hash_layer:
            probs, idx, _ = self._hash_route(logits, input_ids)
            self._apply_expert_bias(idx, padding_mask)
            return probs, idx
        if cfg.moe_z_loss_coeff:
            z = moe_ops.z_loss(logits, cfg.moe_z_loss_coeff)
            # the mean is over this rank's tokens: where the tokens are split over ranks (sequence and context
            # parallelism) the term added to the graph is this rank's share of the mean over all of them
            tp = ps.get_world_size('tp')
            share = (tp if (cfg.sequence_parallel and tp > 1) else 1) * ps.get_world_size('cp')
            logits = moe_ops.MoEAuxLossAutoScaler.apply(logits, z / share if share > 1 else z)
            _track('z_loss', z / cfg.moe_z_loss_coeff)
        probs, idx, scores = moe_ops.topk_routing(
            logits, self.topk, cfg.moe_router_score_function, cfg.moe_router_pre_softmax, cfg.moe_router_num_groups,
            cfg.moe_router_group_topk, cfg.moe_router_topk_scaling_factor, self.expert_bias)
        self._apply_expert_bias(idx, padding_mask)
        lb = cfg.moe_router_load_balancing_type
        coeff = cfg.moe_aux_loss_coeff
        if self.training and coeff and lb in ('aux_loss', 'global_aux_loss', 'seq_aux_loss'):
            valid = None if padding_mask is None else ~padding_mask.reshape(-1)
            if lb == 'seq_aux_loss' and seg_ids is not None:
                split = (cfg.sequence_parallel or cfg.context_parallel_size > 1) and ps.get_world_size('tp_cp') > 1
                aux = moe_ops.seq_aux_loss(scores, idx, seg_ids, num_seqs, self.topk, coeff,
                                           ps.get_group('tp_cp') if split else None)
            else:
                sc = scores if valid is None else scores * valid[:, None]
                counts = moe_ops.tokens_per_expert(idx, self.num_experts, valid)
                ntok = torch.tensor(float(scores.shape[0]), device=x.device) if valid is None else valid.sum().float()
                group = 'tp_dp_cp' if lb == 'global_aux_loss' else ('tp_cp' if cfg.sequence_parallel or
                                                                    cfg.context_parallel_size > 1 else None)
                if group is not None and ps.get_world_size(group) > 1:
                    # f_e uses the counts of the whole (sub)sequence group; P_e stays local (its gradient is local)
                    packed = torch.cat([counts, ntok.view(1)])
                    dist.all_reduce(packed, group=ps.get_group(group))
                    n = ps.get_world_size(group)
                    counts, ntok_all = packed[:-1], packed[-1]
                    ntok_mb = _micro_batch_tokens(cfg, ntok, ntok_all, group)
                    aux = coeff * self.num_experts * ((counts / (ntok_all * self.topk)) * (sc.sum(0) / ntok_mb)).sum()
                else:
                    aux = moe_ops.aux_loss(sc, counts, self.topk, coeff, ntok)
            probs = moe_ops.MoEAuxLossAutoScaler.apply(probs, aux)
            _track('load_balancing_loss', aux / coeff)
        return probs, idx


class GroupedLinear(nn.Module):
    """``E_local`` linears as one stacked parameter; forward over an expert-sorted, padded row buffer."""

    def __init__(self, num_local_experts: int, input_size: int, output_size: int, config, parallel_mode: str,
                 bias: bool = False):
        super().__init__()
        n = ps.get_world_size('etp')
        self.parallel_mode = parallel_mode
        if parallel_mode == 'column':
            output_size //= n
            pdim = 1
        else:
            input_size //= n
            pdim = 2
        self.num_local_experts = num_local_experts
        self.weight = nn.Parameter(torch.empty(num_local_experts, output_size, input_size, dtype=config.params_dtype))
        _set_tp_attrs(self.weight, n > 1, pdim, is_expert=True)
        if bias:
            if n > 1:
                raise NotImplementedError('expert biases are not supported together with expert tensor parallelism')
            self.bias = nn.Parameter(torch.zeros(num_local_experts, output_size, dtype=config.params_dtype))
            _set_tp_attrs(self.bias, False, -1, is_expert=True)
        else:
            self.register_parameter('bias', None)

    def row_bias(self, offsets: torch.Tensor, rows: int, row_scale=None) -> torch.Tensor:
        """``[rows, out]``: every row's expert bias (rows of segment ``e`` are ``offsets[e]:offsets[e+1]``; padding
        rows get the bias of their segment, which nothing reads), optionally scaled per row."""
        eid = torch.searchsorted(offsets[1:].to(torch.int64).contiguous(), torch.arange(rows, device=offsets.device),
                                 right=True).clamp(max=self.num_local_experts - 1)
        b = self.bias[eid]
        return b if row_scale is None else b * row_scale[:, None].to(b.dtype)

    def __getattr__(self, name):
        m = re.fullmatch(r'weight(\d+)', name)
        if m is not None:
            return super().__getattr__('weight')[int(m.group(1))]
        return super().__getattr__(name)

    def forward(self, x, offsets, bias_scale=None):
        y = _GroupedLinearFn.apply(x, self.weight, offsets)
        if self.bias is not None:
            y = y + self.row_bias(offsets, y.shape[0], bias_scale)
        return y


class _GroupedLinearFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, offsets):
        ctx.save_for_backward(x, weight, offsets)
        return gemm.grouped_mm_nt(x, weight, offsets)

    @staticmethod
    def backward(ctx, dy):
        x, weight, offsets = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm.grouped_mm_nn(dy, weight, offsets) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(weight, 'main_grad', None)
            if mg is not None:
                gemm.grouped_mm_tn(dy, x, offsets, out=mg, accumulate=True)
                hook = getattr(weight, 'grad_ready_hook', None)
                if hook is not None:
                    hook()
            else:
                dw = gemm.grouped_mm_tn(dy, x, offsets, out_dtype=weight.dtype)
        return dx, dw, None


class GroupedMLP(nn.Module):
    """All local experts: grouped fc1 -> gated activation (weighted by the routing prob) -> grouped fc2."""

    def __init__(self, config, num_local_experts: int):
        super().__init__()
        self.config = config
        f = config.moe_ffn_hidden_size
        mult = 2 if config.gated_linear_unit else 1
        b = bool(config.add_bias_linear)
        self.linear_fc1 = GroupedLinear(num_local_experts, config.hidden_size, f * mult, config, 'column', bias=b)
        if config.gated_linear_unit:
            for prm in (self.linear_fc1.weight, self.linear_fc1.bias):
                if prm is not None:
                    prm.partition_stride = 2          # [gate shard; up shard] on the output dim
        self.linear_fc2 = GroupedLinear(num_local_experts, f, config.hidden_size, config, 'row', bias=b)
        self.kind = 'swiglu' if config.swiglu else ('quick_geglu' if config.quick_geglu else 'geglu_tanh')

    def forward(self, x, offsets, row_probs=None):
        cfg = self.config
        h = self.linear_fc1(x, offsets)
        if cfg.gated_linear_unit:
            h = glu(h, self.kind, row_probs, cfg.activation_func_clamp_value or 0.0, cfg.glu_linear_offset)
        else:
            h = cfg.activation_func(h)
            if row_probs is not None:
                h = h * row_probs[:, None].to(h.dtype)
        # the routing probability multiplies the expert's whole output, its output bias included
        return self.linear_fc2(h, offsets, row_probs)


class SharedExpertMLP(nn.Module):
    """Always-on expert beside the routed ones, optionally gated by ``sigmoid(x . gate_weight)``."""

    def __init__(self, config, intermediate_size: int):
        super().__init__()
        self.config = config
        mult = 2 if config.gated_linear_unit else 1
        self.linear_fc1 = ColumnParallelLinear(config.hidden_size, intermediate_size * mult, config,
                                               bias=config.add_bias_linear)
        self.linear_fc2 = RowParallelLinear(intermediate_size, config.hidden_size, config, bias=config.add_bias_linear)
        if config.gated_linear_unit:
            for prm in (self.linear_fc1.weight, self.linear_fc1.bias):
                if prm is not None:
                    prm.partition_stride = 2
        if config.moe_shared_expert_gate:
            self.gate_weight = nn.Parameter(torch.empty(1, config.hidden_size, dtype=config.params_dtype))
            mark_sequence_parallel(self.gate_weight, config)
        else:
            self.register_parameter('gate_weight', None)
        self.kind = 'swiglu' if config.swiglu else ('quick_geglu' if config.quick_geglu else 'geglu_tanh')

    def forward(self, x):
        cfg = self.config
        h = self.linear_fc1(x)
        if cfg.gated_linear_unit:
            h = glu(h, self.kind, None, cfg.activation_func_clamp_value or 0.0, cfg.glu_linear_offset)
        else:
            h = cfg.activation_func(h)
        y = self.linear_fc2(h)
        if self.gate_weight is not None:
            g = torch.sigmoid(torch.nn.functional.linear(x.float(), self.gate_weight.float()))
            y = (y.float() * g).to(y.dtype)
        return y


class MoELayer(nn.Module):

    def __init__(self, config, layer_number: int = 1):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        self.ep = ps.get_world_size('ep')
        self.ep_rank = ps.get_rank_in('ep') if self.ep > 1 else 0
        self.num_experts = config.num_moe_experts
        assert self.num_experts % self.ep == 0
        self.num_local_experts = self.num_experts // self.ep
        # the first ``moe_n_hash_layers`` MoE layers of the model route by token id
        moe_before = sum(config.moe_layer_pattern()[:max(0, min(layer_number, config.num_layers) - 1)])
        self.router = TopKRouter(config, is_hash_layer=moe_before < (config.moe_n_hash_layers or 0))
        self.experts = GroupedMLP(config, self.num_local_experts)
        if config.moe_shared_expert_intermediate_size:
            self.shared_experts = SharedExpertMLP(config, config.moe_shared_expert_intermediate_size)
        else:
            self.shared_experts = None
        self.apply_probs_on_input = bool(config.moe_apply_probs_on_input)
        self._fused = None

    # -- hooks for families whose router does not look at the expert input itself
    def _router_input(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def _post_route(self, probs: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        return probs

    # -- dispatch over the EP group with torch.distributed (baseline; host-synchronised split sizes)
    def _dispatch_nccl(self, x, probs, idx):
        T, k = idx.shape
        E, El, ep = self.num_experts, self.num_local_experts, self.ep
        flat_e = idx.reshape(-1)
        src_token = torch.arange(T, device=x.device).repeat_interleave(k)
        order = torch.argsort(flat_e, stable=True)              # copies sorted by global expert = by dest rank
        send = x.index_select(0, src_token[order])
        send_e = flat_e[order]
        send_p = probs.reshape(-1)[order]
        counts = torch.bincount(flat_e, minlength=E)
        all_counts = torch.empty(ep * E, dtype=counts.dtype, device=x.device)     # flat: gloo wants 1-D buffers here
        dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=ps.get_group('ep'))
        all_counts = all_counts.view(ep, E)
        in_splits = counts.view(ep, El).sum(1).tolist()                                   # host sync
        out_splits = all_counts[:, self.ep_rank * El:(self.ep_rank + 1) * El].sum(1).tolist()
        recv = M.all_to_all(send, out_splits, in_splits, 'ep')
        recv_e = M.all_to_all_single(send_e.contiguous(), out_splits, in_splits, 'ep') - self.ep_rank * El
        recv_p = M.all_to_all(send_p.contiguous().view(-1, 1), out_splits, in_splits, 'ep').view(-1)
        return recv, recv_e, recv_p, (order, src_token, in_splits, out_splits)

    def _experts_nccl(self, x: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """Permute / exchange / grouped experts / combine through torch and NCCL (baseline and CPU path)."""
        T = x.shape[0]
        k = idx.shape[1]
        if self.ep == 1:
            src_token = torch.arange(T, device=x.device).repeat_interleave(k)
            dest, offsets, cap = moe_ops.permute_plan(idx.reshape(-1), self.num_local_experts)
            xp = moe_ops.permute(x, src_token, dest, cap)
            pflat = probs.reshape(-1)
            if self.apply_probs_on_input:
                xp = _scale_rows(xp, dest, pflat, cap)
                row_probs = None
            else:
                row_probs = _scatter_rows(pflat, dest, cap)
            yp = self.experts(xp, offsets, row_probs)
            return moe_ops.unpermute(yp, src_token, dest, T, None)
        recv, recv_e, recv_p, (order, src_token, in_splits, out_splits) = self._dispatch_nccl(x, probs, idx)
        R = recv.shape[0]
        dest, offsets, cap = moe_ops.permute_plan(recv_e, self.num_local_experts)
        ar = torch.arange(R, device=x.device)
        xp = moe_ops.permute(recv, ar, dest, cap)
        if self.apply_probs_on_input:
            xp = _scale_rows(xp, dest, recv_p, cap)
            row_probs = None
        else:
            row_probs = _scatter_rows(recv_p, dest, cap)
        yp = self.experts(xp, offsets, row_probs)
        back = moe_ops.unpermute(yp, ar, dest, R, None)          # rows back in arrival order
        ret = M.all_to_all(back, in_splits, out_splits, 'ep')    # rows in `order`
        return moe_ops.unpermute(ret, src_token[order], torch.arange(ret.shape[0], device=x.device), T, None)

    def _forward_fused(self, x, padding_mask, seg_ids, num_seqs, input_ids=None):
        """Router, exchange and combine on the in-tree kernels (``layers/moe_fused.py``)."""
        from . import moe_fused as F
        cfg = self.config
        r = self.router
        T, H = x.shape
        if self._fused is None:
            self._fused = F.FusedMoEDispatcher(cfg, self.num_local_experts)
        st = self._fused.begin(T, H, x.device)
        lb = cfg.moe_router_load_balancing_type
        kernel_router = (F.router_supported(self.num_experts, r.topk, cfg.moe_router_num_groups)
                         and not r.is_hash_layer
                         and not (self.training and cfg.moe_aux_loss_coeff and lb == 'seq_aux_loss')
                         and not cfg.moe_z_loss_coeff
                         # softmax scores with a selection bias (Ernie-4.5) stay on the torch router
                         and not (cfg.moe_router_score_function != 'sigmoid' and r.expert_bias is not None))
        if kernel_router:
            logits = r.gating(self._router_input(x)).float()
            valid = None if padding_mask is None else ~padding_mask.reshape(-1)
            sigmoid = cfg.moe_router_score_function == 'sigmoid'
            renorm = (not cfg.moe_router_pre_softmax) and (not sigmoid or r.topk > 1)
            bias = r.expert_bias if (sigmoid and r.expert_bias is not None) else None
            probs, idx, score_sum, counts = self._fused.route(st, logits, bias, valid, sigmoid, renorm,
                                                              cfg.moe_router_num_groups, cfg.moe_router_group_topk,
                                                              cfg.moe_router_topk_scaling_factor)
            if r.enable_expert_bias and torch.is_grad_enabled():
                with torch.no_grad():
                    r.local_tokens_per_expert += counts.float()
            coeff = cfg.moe_aux_loss_coeff
            if self.training and coeff and lb in ('aux_loss', 'global_aux_loss'):
                ntok = torch.tensor(float(T), device=x.device) if valid is None else valid.sum().float()
                cnt = counts.float()
                group = 'tp_dp_cp' if lb == 'global_aux_loss' else ('tp_cp' if cfg.sequence_parallel or
                                                                    cfg.context_parallel_size > 1 else None)
                ntok_all = ntok
                if group is not None and ps.get_world_size(group) > 1:
                    packed = torch.cat([cnt, ntok.view(1)])
                    dist.all_reduce(packed, group=ps.get_group(group))
                    cnt, ntok_all = packed[:-1], packed[-1]
                ntok_p = _micro_batch_tokens(cfg, ntok, ntok_all, group) if group is not None and \
                    ps.get_world_size(group) > 1 else ntok
                aux = coeff * self.num_experts * ((cnt / (ntok_all * r.topk)) * (score_sum / ntok_p)).sum()
                probs = moe_ops.MoEAuxLossAutoScaler.apply(probs, aux)
                _track('load_balancing_loss', aux / coeff)
        else:
            probs, idx = r(self._router_input(x), padding_mask, seg_ids, num_seqs, input_ids)
            self._fused.publish_routing(st, idx)
            idx = idx.to(torch.int32)
        probs = self._post_route(probs, idx)
        if F.pull_gemm_supported(self.experts, cfg, self.num_local_experts, H):
            y = self._fused.experts_fused(st, x, probs, idx, self.experts)
            if self.shared_experts is not None:
                y = y + self.shared_experts(x)
            return y
        xp, row_probs = self._fused.dispatch(st, x, probs, idx)
        if self.apply_probs_on_input:
            xp = (xp.float() * row_probs[:, None]).to(xp.dtype)
            row_probs = None
        yp = self.experts(xp, st.seg_off, row_probs)
        y = self._fused.combine(st, yp)
        if self.shared_experts is not None:
            y = y + self.shared_experts(x)
        return y

    def forward(self, x: torch.Tensor, padding_mask: Optional[torch.Tensor] = None, seg_ids=None, num_seqs=None,
                input_ids: Optional[torch.Tensor] = None):
        """``x [T_local, H]`` -> ``[T_local, H]``.  ``input_ids`` (this rank's token ids) is only read by hash-routed
        layers."""
        cfg = self.config
        T, H = x.shape
        from . import moe_fused
        if moe_fused.available(x) and ps.get_world_size('etp') == 1 and H % 8 == 0:
            return self._forward_fused(x, padding_mask, seg_ids, num_seqs, input_ids)
        probs, idx = self.router(self._router_input(x), padding_mask, seg_ids, num_seqs, input_ids)
        probs = self._post_route(probs, idx)
        etp = ps.get_world_size('etp')
        x_in = x
        if etp > 1:
            # Expert tensor parallelism: every rank of the group holds a slice of each local expert's FFN, so all of
            # them process the group's tokens and their partial outputs are summed.  Routing is computed once per
            # token (on the rank that owns it) and shared.
            sp = cfg.sequence_parallel and ps.get_world_size('tp') > 1
            if sp:      # tokens are sharded over the group: gather them (gradient: reduce-scatter of the partials)
                x_in = M.gather_from_sequence_parallel_region(x, 'etp', tensor_parallel_output_grad=True)
                probs = M.gather_from_sequence_parallel_region(probs, 'etp', tensor_parallel_output_grad=True)
                idx = M.all_gather_dim0(idx.contiguous(), 'etp')
            else:       # tokens are replicated: identity forward, gradients of the partial paths are summed
                x_in = M.copy_to_tensor_model_parallel_region(x, 'etp')
                probs = M.copy_to_tensor_model_parallel_region(probs, 'etp')
        y = self._experts_nccl(x_in, probs, idx)
        if etp > 1:
            y = M.reduce_scatter_to_sequence_parallel_region(y, 'etp') if sp else \
                M.reduce_from_tensor_model_parallel_region(y, 'etp')
        if self.shared_experts is not None:
            y = y + self.shared_experts(x)
        return y


class _ScatterRows(torch.autograd.Function):
    """``out[dest[i]] = v[i]`` into a zero vector of length ``cap`` (per-row routing probabilities)."""

    @staticmethod
    def forward(ctx, v, dest, cap):
        out = torch.zeros(cap, dtype=torch.float32, device=v.device)
        out.index_copy_(0, dest, v.float())
        ctx.save_for_backward(dest)
        ctx.dtype = v.dtype
        return out

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        return g.index_select(0, dest).to(ctx.dtype), None, None


def _scatter_rows(v, dest, cap):
    return _ScatterRows.apply(v, dest, cap)


def _scale_rows(xp, dest, v, cap):
    return (xp.float() * _scatter_rows(v, dest, cap)[:, None]).to(xp.dtype)
