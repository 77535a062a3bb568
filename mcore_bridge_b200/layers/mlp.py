"""Dense feed-forward block: (fused-norm) fc1 -> gated activation -> fc2."""
from __future__ import annotations

import torch
from torch import nn

from ..ops.activation import glu
from .linear import ColumnParallelLinear, LayerNormColumnParallelLinear, RowParallelLinear


class MLP(nn.Module):

    def __init__(self, config, ffn_hidden_size: int = None, fuse_input_norm: bool = True):
        super().__init__()
        self.config = config
        f = ffn_hidden_size or config.ffn_hidden_size
        mult = 2 if config.gated_linear_unit else 1
        cls = LayerNormColumnParallelLinear if fuse_input_norm else ColumnParallelLinear
        self.linear_fc1 = cls(config.hidden_size, f * mult, config, bias=config.add_bias_linear)
        self.linear_fc2 = RowParallelLinear(f, config.hidden_size, config, bias=config.add_bias_linear)
        if config.gated_linear_unit:
            # the local shard is [gate shard; up shard]: two interleaved partitions of the output dim
            for prm in (self.linear_fc1.weight, self.linear_fc1.bias):
                if prm is not None:
                    prm.partition_stride = 2
        self.kind = 'swiglu' if config.swiglu else ('quick_geglu' if config.quick_geglu else 'geglu_tanh')

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        h = self.linear_fc1(x)
        fc2 = self.linear_fc2
        if cfg.gated_linear_unit and type(fc2) is RowParallelLinear and fc2.bias is None and not fc2.spec.fp8 \
                and getattr(cfg, 'lean_activations', True):
            from ..parallel import state as ps
            from ..ops import fused_mlp
            if ps.get_world_size(fc2.group) == 1 and fused_mlp.usable(h, fc2.weight) and (h.shape[-1] // 2) % 8 == 0:
                from ..ops.activation import KINDS
                return fused_mlp.glu_linear(h, fc2.weight, KINDS[self.kind], cfg.activation_func_clamp_value or 0.0,
                                            cfg.glu_linear_offset)
        if cfg.gated_linear_unit:
            h = glu(h, self.kind, None, cfg.activation_func_clamp_value or 0.0, cfg.glu_linear_offset)
        else:
            h = cfg.activation_func(h)
        return self.linear_fc2(h)
