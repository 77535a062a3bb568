"""Tensor-parallel linear modules.

Module and parameter names follow the Megatron conventions the weight bridge and LoRA ``target_modules``
are written against (reference ``src/mcore_bridge/bridge/gpt_bridge.py:124-163``): ``weight``, ``bias``,
and ``layer_norm_weight`` / ``layer_norm_bias`` for a linear with the preceding norm folded in.
Parameters carry ``tensor_model_parallel`` / ``partition_dim`` attributes describing their sharding.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..ops.linear import LinearSpec, linear
from ..ops.norm import layernorm_ref, rmsnorm
from ..parallel import state as ps
from .norm import mark_sequence_parallel


def _set_tp_attrs(p: nn.Parameter, is_parallel: bool, dim: int, is_expert: bool = False):
    p.tensor_model_parallel = is_parallel
    p.partition_dim = dim if is_parallel else -1
    p.partition_stride = 1
    p.allreduce = not is_expert  # expert params are reduced over the expert-data-parallel group instead
    p.is_expert = is_expert


class _LinearBase(nn.Module):

    def _group(self, is_expert: bool) -> str:
        return 'etp' if is_expert else 'tp'


def _fp8_default(config) -> bool:
    """Block-scaled fp8 GEMMs for the decoder's linear layers when the config asks for fp8 training with the
    blockwise recipe (128 x 128 weight blocks, 1 x 128 activation blocks)."""
    return getattr(config, 'fp8', None) is not None and getattr(config, 'fp8_recipe', None) in (None, 'blockwise')


class ColumnParallelLinear(_LinearBase):
    """``y = x W^T + b`` with ``W [out/tp, in]``."""

    def __init__(self, input_size: int, output_size: int, config, bias: bool = False, gather_output: bool = False,
                 is_expert: bool = False, skip_bias_add: bool = False, tp_group: Optional[str] = None,
                 sequence_parallel: Optional[bool] = None, params_dtype=None, fp8: Optional[bool] = None):
        super().__init__()
        self.config = config
        self.group = tp_group or self._group(is_expert)
        n = ps.get_world_size(self.group)
        assert output_size % n == 0, f'output size {output_size} not divisible by TP {n}'
        self.input_size, self.output_size = input_size, output_size
        self.output_size_per_partition = output_size // n
        self.is_expert = is_expert
        self.gather_output = gather_output
        self.sequence_parallel = config.sequence_parallel if sequence_parallel is None else sequence_parallel
        if n == 1:
            self.sequence_parallel = False
        dtype = params_dtype or config.params_dtype
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size, dtype=dtype))
        _set_tp_attrs(self.weight, n > 1, 0, is_expert)
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=dtype))
            _set_tp_attrs(self.bias, n > 1, 0, is_expert)
        else:
            self.register_parameter('bias', None)
        self.spec = LinearSpec(mode='column', sequence_parallel=self.sequence_parallel, group=self.group,
                               gather_output=gather_output, fp8=_fp8_default(config) if fp8 is None else fp8)

    def forward(self, x):
        return linear(x, self.weight, self.bias, self.spec)

    def extra_repr(self):
        return (f'in={self.input_size}, out={self.output_size_per_partition} (of {self.output_size}), '
                f'bias={self.bias is not None}, sp={self.sequence_parallel}')


class LayerNormColumnParallelLinear(ColumnParallelLinear):
    """Norm folded into the following column-parallel linear (``layer_norm_weight``).

    The norm runs on the local (sequence-sharded) tokens, then the fused all-gather -> GEMM follows.
    ``forward`` can also return the normalised input, which LoRA adapters consume
    (reference ``src/mcore_bridge/tuners/lora.py:378-414``).
    """

    def __init__(self, input_size: int, output_size: int, config, bias: bool = False, **kw):
        super().__init__(input_size, output_size, config, bias=bias, **kw)
        dtype = config.params_dtype
        self.eps = config.layernorm_epsilon
        self.zero_centered = config.layernorm_zero_centered_gamma
        self.normalization = config.normalization
        init = torch.zeros if self.zero_centered else torch.ones
        self.layer_norm_weight = nn.Parameter(init(input_size, dtype=dtype))
        mark_sequence_parallel(self.layer_norm_weight, config)
        if self.normalization == 'LayerNorm':
            self.layer_norm_bias = nn.Parameter(torch.zeros(input_size, dtype=dtype))
            mark_sequence_parallel(self.layer_norm_bias, config)
        else:
            self.register_parameter('layer_norm_bias', None)
        self.return_layernorm_output = False

    def norm(self, x):
        if self.normalization == 'LayerNorm':
            w = self.layer_norm_weight + 1.0 if self.zero_centered else self.layer_norm_weight
            return layernorm_ref(x, w, self.layer_norm_bias, self.eps)
        return rmsnorm(x, self.layer_norm_weight, self.eps, self.zero_centered)

    def _lean(self, x) -> bool:
        """Single-rank RMSNorm path that does not keep the normalised activation (``ops/fused_mlp.py``)."""
        if self.return_layernorm_output or self.bias is not None or self.spec.fp8 or self.gather_output:
            return False
        if self.normalization == 'LayerNorm' or ps.get_world_size(self.group) > 1 or self.input_size > 16384:
            return False
        if not getattr(self.config, 'lean_activations', True):
            return False
        from ..ops import fused_mlp
        return fused_mlp.usable(x, self.weight) and self.layer_norm_weight.dtype == torch.bfloat16

    def forward(self, x):
        if self._lean(x):
            from ..ops import fused_mlp
            return fused_mlp.norm_linear(x, self.layer_norm_weight, self.weight, self.eps, self.zero_centered)
        xn = self.norm(x)
        y = linear(xn, self.weight, self.bias, self.spec)
        if self.return_layernorm_output:
            return y, xn
        return y


class RowParallelLinear(_LinearBase):
    """``y = x W^T + b`` with ``W [out, in/tp]``; output reduce-scattered (SP) or all-reduced."""

    def __init__(self, input_size: int, output_size: int, config, bias: bool = False, input_is_parallel: bool = True,
                 is_expert: bool = False, tp_group: Optional[str] = None, sequence_parallel: Optional[bool] = None,
                 params_dtype=None, fp8: Optional[bool] = None):
        super().__init__()
        self.config = config
        self.group = tp_group or self._group(is_expert)
        n = ps.get_world_size(self.group)
        assert input_size % n == 0, f'input size {input_size} not divisible by TP {n}'
        self.input_size, self.output_size = input_size, output_size
        self.input_size_per_partition = input_size // n
        self.is_expert = is_expert
        self.sequence_parallel = config.sequence_parallel if sequence_parallel is None else sequence_parallel
        if n == 1:
            self.sequence_parallel = False
        dtype = params_dtype or config.params_dtype
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition, dtype=dtype))
        _set_tp_attrs(self.weight, n > 1, 1, is_expert)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=dtype))
            _set_tp_attrs(self.bias, False, -1, is_expert)
            mark_sequence_parallel(self.bias, config)
        else:
            self.register_parameter('bias', None)
        self.spec = LinearSpec(mode='row', sequence_parallel=self.sequence_parallel, group=self.group,
                               fp8=_fp8_default(config) if fp8 is None else fp8)

    def forward(self, x):
        return linear(x, self.weight, self.bias, self.spec)

    def extra_repr(self):
        return (f'in={self.input_size_per_partition} (of {self.input_size}), out={self.output_size}, '
                f'bias={self.bias is not None}, sp={self.sequence_parallel}')


class ReplicatedLinear(nn.Module):
    """A plain linear replicated on every TP rank (router gates, small heads)."""

    def __init__(self, input_size: int, output_size: int, config, bias: bool = False, params_dtype=None,
                 sequence_parallel_grad: bool = True):
        super().__init__()
        dtype = params_dtype or config.params_dtype
        self.weight = nn.Parameter(torch.empty(output_size, input_size, dtype=dtype))
        _set_tp_attrs(self.weight, False, -1)
        if sequence_parallel_grad:
            mark_sequence_parallel(self.weight, config)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=dtype))
            if sequence_parallel_grad:
                mark_sequence_parallel(self.bias, config)
        else:
            self.register_parameter('bias', None)

    def forward(self, x):
        return linear(x, self.weight, self.bias, LinearSpec())
