"""Normalisation modules (RMSNorm with optional zero-centred gamma, LayerNorm)."""
from __future__ import annotations

import torch
from torch import nn

from ..ops.norm import layernorm_ref, rmsnorm


def mark_sequence_parallel(param: torch.nn.Parameter, config) -> None:
    """Norm weights are replicated over TP; under sequence parallelism each rank sees only its tokens,
    so their gradients must be summed over the TP group (the optimizer does it for flagged params)."""
    param.sequence_parallel = bool(config.sequence_parallel)


class Norm(nn.Module):
    """RMSNorm or LayerNorm over the last dimension; ``config.layernorm_zero_centered_gamma`` stores gamma-1."""

    def __init__(self, config, hidden_size: int, eps: float = None, zero_centered: bool = None,
                 normalization: str = None, sequence_parallel_grad: bool = True):
        super().__init__()
        self.config = config
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.zero_centered = config.layernorm_zero_centered_gamma if zero_centered is None else zero_centered
        self.normalization = normalization or config.normalization
        dtype = config.params_dtype
        init = torch.zeros if self.zero_centered else torch.ones
        self.weight = nn.Parameter(init(hidden_size, dtype=dtype))
        if self.normalization == 'LayerNorm':
            self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype))
        else:
            self.bias = None
        if sequence_parallel_grad:
            mark_sequence_parallel(self.weight, config)
            if self.bias is not None:
                mark_sequence_parallel(self.bias, config)

    def forward(self, x):
        if self.normalization == 'LayerNorm':
            w = self.weight + 1.0 if self.zero_centered else self.weight
            return layernorm_ref(x, w, self.bias, self.eps)
        return rmsnorm(x, self.weight, self.eps, self.zero_centered)

    def extra_repr(self):
        return f'{self.weight.shape[0]}, eps={self.eps}, zero_centered={self.zero_centered}, {self.normalization}'
