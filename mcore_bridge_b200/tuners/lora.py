"""LoRA over the tensor-parallel linears, grouped expert linears and the MoE router.

``LoraParallelLinear`` wraps a base layer and adds ``scaling * B(A(dropout(x)))``.  Placement of the low-rank
factors follows the base layer's sharding (parity: reference ``src/mcore_bridge/tuners/lora.py:178-271``):

* column-parallel base  ->  ``A`` replicated ``[r, in]``, ``B`` column-parallel ``[out/tp, r]``.  Under sequence
  parallelism ``A`` runs on the local tokens and only the rank-``r`` activations are all-gathered.
* row-parallel base     ->  ``A`` row-parallel ``[r, in/tp]``, ``B`` replicated ``[out, r]``; the rank-``r``
  partial sums are reduce-scattered (sequence parallel) or all-reduced.
* grouped (expert) base ->  stacked ``A [E, r, in]``, ``B [E, out, r]`` run with the grouped GEMM and the same
  per-expert row offsets as the base layer.
* router                ->  plain ``A``/``B`` added to the gate logits.

A fused-norm base layer hands its normalised input to the adapter (``return_layernorm_output``), as the
reference does at ``:378-414``.  ``merge`` / ``unmerge`` / ``get_delta_weight`` fold the adapter into the base
weight shard.  DoRA and expert tensor parallelism are rejected like in the reference (``:116-132``).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ..layers.linear import LayerNormColumnParallelLinear, ReplicatedLinear, RowParallelLinear, _set_tp_attrs
from ..layers.moe import GroupedLinear, TopKRouter, _GroupedLinearFn
from ..ops.linear import LinearSpec, linear
from ..parallel import mappings as M
from ..parallel import state as ps
from ..parallel.random import get_rng_tracker


class _AccumulateLoraB(torch.autograd.Function):
    """``result += scaling * h @ B^T`` written by the second adapter GEMM straight into the base layer's output
    (the GEMM epilogue reads and adds the tile it is about to store), instead of materialising the adapter output
    and adding it in a separate pass over ``[T, N]``."""

    @staticmethod
    def forward(ctx, result, h, b, scaling):
        from ..ops import gemm
        ctx.save_for_backward(h, b)
        ctx.scaling = scaling
        gemm.mm_nt(h, b, out=result, accumulate=True, alpha=scaling)
        ctx.mark_dirty(result)
        return result

    @staticmethod
    def backward(ctx, g):
        from ..ops import gemm
        h, b = ctx.saved_tensors
        g2 = g.reshape(-1, g.shape[-1])
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dh = db = None
        if ctx.needs_input_grad[1]:
            dh = gemm.mm_nn(g2, b, alpha=ctx.scaling).view(*g.shape[:-1], b.shape[1])
        if ctx.needs_input_grad[2]:
            db = gemm.mm_tn(g2, h.reshape(-1, h.shape[-1]), alpha=ctx.scaling, out_dtype=b.dtype)
        return g, dh, db, None


def is_expert_layer(layer) -> bool:
    return bool(getattr(layer, 'is_expert', False)) or isinstance(layer, GroupedLinear)


class _LoraFactor(nn.Module):
    """One low-rank factor: a ``weight`` (2-D, or 3-D stacked per expert) with sharding attributes."""

    def __init__(self, shape, dtype, device, tp_parallel: bool, partition_dim: int, is_expert: bool,
                 sequence_parallel_grad: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(*shape, dtype=dtype, device=device))
        _set_tp_attrs(self.weight, tp_parallel, partition_dim, is_expert)
        if sequence_parallel_grad:
            self.weight.sequence_parallel = True
        else:
            # replicated factor seeing identical activations on every TP rank: average to stay bit-identical
            self.weight.average_gradients_across_tp_domain = not tp_parallel

    def __getattr__(self, name):
        if name.startswith('weight') and name[6:].isdigit():
            return super().__getattr__('weight')[int(name[6:])]
        return super().__getattr__(name)


class LoraParallelLinear(nn.Module):

    def __init__(self, base_layer: nn.Module, adapter_name: str = 'default', r: int = 8, lora_alpha: int = 16,
                 lora_dropout: float = 0.0, fan_in_fan_out: bool = False, init_lora_weights=True,
                 use_rslora: bool = False, use_dora: bool = False, lora_bias: bool = False, **kwargs):
        super().__init__()
        if use_dora:
            raise ValueError(f'{self.__class__.__name__} does not support DoRA yet, please set it to False')
        self.base_layer = base_layer
        self.config = getattr(base_layer, 'config', None)
        self.is_router = isinstance(base_layer, TopKRouter)
        self.is_grouped = isinstance(base_layer, GroupedLinear)
        self.is_parallel_a = isinstance(base_layer, RowParallelLinear) or (
            self.is_grouped and base_layer.parallel_mode == 'row')
        self.is_expert = is_expert_layer(base_layer)
        # a linear replicated over the TP group (MLA down projections, DSA indexer linears): the adapter is replicated
        # too and runs on whatever tokens the layer sees, without any collective
        self.is_replicated = isinstance(base_layer, ReplicatedLinear)
        self.sequence_parallel = bool(getattr(base_layer, 'sequence_parallel', False))
        self.group = 'etp' if self.is_expert else 'tp'
        self.tp_size = ps.get_world_size(self.group)
        if self.is_expert and self.tp_size > 1:
            raise ValueError('Currently, LoRA does not support ETP.')
        self.fan_in_fan_out = fan_in_fan_out
        self.lora_A = nn.ModuleDict()
        self.lora_B = nn.ModuleDict()
        self.lora_dropout = nn.ModuleDict()
        self.r: Dict[str, int] = {}
        self.lora_alpha: Dict[str, int] = {}
        self.scaling: Dict[str, float] = {}
        self.merged_adapters: List[str] = []
        self.disable_adapters = False
        self._active_adapter = adapter_name
        w = base_layer.weight
        if self.is_grouped:
            self.num_gemms, self.out_features, self.in_features = w.shape
        else:
            self.out_features, self.in_features = w.shape
        self.update_layer(adapter_name, r, lora_alpha=lora_alpha, lora_dropout=lora_dropout,
                          init_lora_weights=init_lora_weights, use_rslora=use_rslora, lora_bias=lora_bias)

    # ------------------------------------------------------------------ PEFT-compatible surface
    @property
    def active_adapters(self) -> List[str]:
        a = self._active_adapter
        return [a] if isinstance(a, str) else list(a)

    @property
    def merged(self) -> bool:
        return bool(self.merged_adapters)

    @property
    def weight(self):
        return self.base_layer.weight

    @property
    def bias(self):
        return getattr(self.base_layer, 'bias', None)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            if name == 'base_layer':
                raise
            return getattr(self.base_layer, name)  # layer_norm_weight, sequence_parallel, ...

    def set_adapter(self, names):
        self._active_adapter = names
        act = set(self.active_adapters)
        for key in self.lora_A:
            for p in list(self.lora_A[key].parameters()) + list(self.lora_B[key].parameters()):
                p.requires_grad_(key in act)

    def enable_adapters(self, enabled: bool):
        self.disable_adapters = not enabled

    def update_layer(self, adapter_name, r, *, lora_alpha, lora_dropout=0.0, init_lora_weights=True,
                     use_rslora=False, lora_bias=False, **kwargs):
        if r <= 0:
            raise ValueError(f'`r` should be a positive integer value but the value passed is {r}')
        if lora_bias:
            raise ValueError('lora_bias is not supported')
        self.r[adapter_name] = r
        self.lora_alpha[adapter_name] = lora_alpha
        self.lora_dropout[adapter_name] = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else nn.Identity()
        w = self.base_layer.weight
        dt, dev = w.dtype, w.device
        tp = self.tp_size
        sp = self.sequence_parallel
        if self.is_router:
            a = _LoraFactor((r, self.in_features), dt, dev, False, -1, False, bool(self.config.sequence_parallel))
            b = _LoraFactor((self.out_features, r), dt, dev, False, -1, False, bool(self.config.sequence_parallel))
        elif self.is_grouped:
            # A/B stacked per expert.  Row base: A sees the sharded input; column base: B produces the sharded output.
            a = _LoraFactor((self.num_gemms, r, self.in_features), dt, dev, False, -1, True, False)
            b = _LoraFactor((self.num_gemms, self.out_features, r), dt, dev, False, -1, True, False)
        elif self.is_replicated:
            # gradients follow the base weight: summed over the TP group where every rank sees its own tokens
            # (sequence parallelism), otherwise identical on every rank
            sum_tp = bool(getattr(w, 'sequence_parallel', False))
            a = _LoraFactor((r, self.in_features), dt, dev, False, -1, False, sum_tp)
            b = _LoraFactor((self.out_features, r), dt, dev, False, -1, False, sum_tp)
        elif self.is_parallel_a:
            a = _LoraFactor((r, self.in_features), dt, dev, tp > 1, 1, self.is_expert, False)
            b = _LoraFactor((self.out_features, r), dt, dev, False, -1, self.is_expert, sp)
        else:
            a = _LoraFactor((r, self.in_features), dt, dev, False, -1, self.is_expert, sp)
            b = _LoraFactor((self.out_features, r), dt, dev, tp > 1, 0, self.is_expert, False)
            # rows laid out like the base weight's (a gated MLP keeps [gate shard; up shard] on every rank): sharded
            # checkpoints re-partition the factor with the same stride
            b.weight.partition_stride = int(getattr(w, 'partition_stride', 1))
        self.lora_A[adapter_name] = a
        self.lora_B[adapter_name] = b
        self.scaling[adapter_name] = lora_alpha / math.sqrt(r) if use_rslora else lora_alpha / r
        if init_lora_weights:
            self.reset_lora_parameters(adapter_name, init_lora_weights)
        self.set_adapter(self.active_adapters)

    def _rng_context(self, factor: _LoraFactor):
        """Sharded factors draw from the TP (or expert) stream, replicated ones from the shared stream, so a
        checkpoint-free restart reproduces the same adapter on every layout."""
        tracker = get_rng_tracker()
        import contextlib
        if self.is_expert and 'expert-parallel-rng' in tracker.states:
            return tracker.fork('expert-parallel-rng')
        if getattr(factor.weight, 'tensor_model_parallel', False) and 'model-parallel-rng' in tracker.states:
            return tracker.fork('model-parallel-rng')
        return contextlib.nullcontext()

    @torch.no_grad()
    def reset_lora_parameters(self, adapter_name, init_lora_weights=True):
        if init_lora_weights is False:
            return
        a, b = self.lora_A[adapter_name], self.lora_B[adapter_name]
        with self._rng_context(a):
            if init_lora_weights is True:
                w = a.weight
                for sl in (w if w.dim() == 3 else [w]):
                    nn.init.kaiming_uniform_(sl, a=math.sqrt(5))
            elif str(init_lora_weights).lower() == 'gaussian':
                nn.init.normal_(a.weight, std=1 / self.r[adapter_name])
            else:
                raise ValueError(f'Unknown initialization {init_lora_weights=}')
        b.weight.zero_()

    # ------------------------------------------------------------------ adapter math
    def _lora_dense_a(self, x: torch.Tensor, name: str) -> torch.Tensor:
        """First adapter GEMM and the collective the base layer's parallel mode calls for; returns ``h [.., r]``."""
        a = self.lora_A[name].weight
        x = self.lora_dropout[name](x).to(a.dtype)
        tp, sp = self.tp_size, self.sequence_parallel
        h = linear(x, a, None, LinearSpec())
        if self.is_replicated:
            return h
        if tp > 1 and self.is_parallel_a:                          # partial sums over the input shards
            return M.reduce_scatter_to_sequence_parallel_region(h, self.group) if sp else \
                M.reduce_from_tensor_model_parallel_region(h, self.group)
        if tp > 1:
            return M.gather_from_sequence_parallel_region(h, self.group, tensor_parallel_output_grad=True) if sp \
                else M.copy_to_tensor_model_parallel_region(h, self.group)
        return h

    def _lora_dense(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return linear(self._lora_dense_a(x, name), self.lora_B[name].weight, None, LinearSpec())

    @staticmethod
    def _can_accumulate(result: torch.Tensor, h: torch.Tensor, b: torch.Tensor) -> bool:
        # an alias of another tensor cannot be updated in place under autograd: those cases add out of place
        return (torch.is_tensor(result) and result._base is None and result.dtype == h.dtype == b.dtype
                and result.is_contiguous()
                and result.shape[:-1] == h.shape[:-1] and result.shape[-1] == b.shape[0]
                and (not result.is_cuda or result.dtype == torch.bfloat16))

    def _lora_grouped(self, x: torch.Tensor, offsets: torch.Tensor, name: str) -> torch.Tensor:
        a, b = self.lora_A[name].weight, self.lora_B[name].weight
        x = self.lora_dropout[name](x).to(a.dtype)
        r = a.shape[1]
        if r % 64 != 0 and x.is_cuda:
            # the grouped input-gradient kernel contracts over r in 64-wide steps: small ranks use padded factors
            pad = (-r) % 64
            a = torch.nn.functional.pad(a, (0, 0, 0, pad))
            b = torch.nn.functional.pad(b, (0, pad))
        h = _GroupedLinearFn.apply(x, a, offsets)
        return _GroupedLinearFn.apply(h, b, offsets)

    def forward(self, x: torch.Tensor, *args: Any, **kwargs: Any):
        if self.disable_adapters and self.merged:
            self.unmerge()
        use = not self.disable_adapters and not self.merged
        base = self.base_layer
        if self.is_router:
            return base(x, *args, **kwargs) if not use else self._router_forward(x, *args, **kwargs)
        # a caller that also wants the normalised input of a fused norm + linear (MLA hands it to the DSA indexer) sets
        # ``return_layernorm_output`` on whatever module sits in the slot: honoured here like on the bare layer
        want_norm = bool(self.__dict__.get('return_layernorm_output', False)) and \
            isinstance(base, LayerNormColumnParallelLinear)
        if isinstance(base, LayerNormColumnParallelLinear):
            if not use and not want_norm:
                base.return_layernorm_output = False
                return base(x)
            base.return_layernorm_output = True
            try:
                result, x = base(x)
            finally:
                base.return_layernorm_output = False
        else:
            result = base(x, *args, **kwargs)
        if not use:
            return (result, x) if want_norm else result
        for name in self.active_adapters:
            if name not in self.lora_A:
                continue
            if self.is_grouped:
                delta = self._lora_grouped(x, args[0] if args else kwargs['offsets'], name)
            else:
                h, b = self._lora_dense_a(x, name), self.lora_B[name].weight
                # a column-parallel base that hands out its gathered output: the adapter's columns are gathered too
                gathered = self.tp_size > 1 and bool(getattr(base, 'gather_output', False))
                if not gathered and self._can_accumulate(result, h, b):
                    result = _AccumulateLoraB.apply(result, h, b, float(self.scaling[name]))
                    continue
                delta = linear(h, b, None, LinearSpec())
                if gathered:
                    delta = M.gather_from_tensor_model_parallel_region(delta, self.group)
            result = result + delta * self.scaling[name]
        result = result.to(x.dtype) if result.dtype != x.dtype and x.is_floating_point() else result
        return (result, x) if want_norm else result

    def effective_weight(self) -> torch.Tensor:
        """Base weight plus the active adapters' ``scaling * B @ A`` (differentiable in the factors): for callers that
        use the matrix itself instead of calling the layer (weight-absorbed MLA)."""
        w = self.base_layer.weight
        if self.disable_adapters or self.merged:
            return w
        for name in self.active_adapters:
            if name in self.lora_A:
                w = w + self.get_delta_weight(name)
        return w

    def _router_forward(self, x, *args, **kwargs):
        """Adds the adapter to the gate logits by swapping ``gating`` for the duration of the call
        (reference ``src/mcore_bridge/tuners/lora.py:341-371``)."""
        base = self.base_layer
        orig = base.gating

        def gating(inp):
            logits = orig(inp)
            for name in self.active_adapters:
                if name in self.lora_A:
                    a, b = self.lora_A[name].weight, self.lora_B[name].weight
                    h = torch.nn.functional.linear(self.lora_dropout[name](inp).to(a.dtype), a)
                    logits = logits + (torch.nn.functional.linear(h, b) * self.scaling[name]).to(logits.dtype)
            return logits

        base.gating = gating
        try:
            return base(x, *args, **kwargs)
        finally:
            base.gating = orig

    # ------------------------------------------------------------------ merging
    def get_delta_weight(self, adapter: str) -> torch.Tensor:
        """``scaling * B @ A`` for this rank's shard of the base weight."""
        a, b = self.lora_A[adapter].weight.float(), self.lora_B[adapter].weight.float()
        delta = torch.matmul(b, a) * self.scaling[adapter]
        return delta.to(self.base_layer.weight.dtype)

    @torch.no_grad()
    def merge(self, safe_merge: bool = False, adapter_names: Optional[List[str]] = None) -> None:
        for name in (adapter_names or self.active_adapters):
            if name not in self.lora_A or name in self.merged_adapters:
                continue
            delta = self.get_delta_weight(name)
            if safe_merge:
                merged = self.base_layer.weight + delta
                if not torch.isfinite(merged).all():
                    raise ValueError(f'NaNs detected in the merged weights. The adapter {name} seems to be broken')
                self.base_layer.weight.copy_(merged)
            else:
                self.base_layer.weight.add_(delta)
            self.merged_adapters.append(name)

    @torch.no_grad()
    def unmerge(self) -> None:
        while self.merged_adapters:
            name = self.merged_adapters.pop()
            if name in self.lora_A:
                self.base_layer.weight.sub_(self.get_delta_weight(name))

    def __repr__(self):
        return 'lora.' + super().__repr__()
