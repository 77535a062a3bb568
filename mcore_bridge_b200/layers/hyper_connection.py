"""Manifold-constrained hyper-connections (mHC): ``n`` residual streams instead of one.

The block keeps ``n`` copies of the residual (``[T, n * C]``, stream-major).  Around every sub-layer (attention, MLP)
a ``HyperConnection`` computes, per token and from the token's own streams, three small maps:

* ``pre``  ``[n]``      how the streams are mixed into the sub-layer's input:  ``x = sum_i pre[i] * s_i``
* ``post`` ``[n]``      how the sub-layer's output is written back to each stream
* ``res``  ``[n, n]``   how the streams are mixed among themselves; projected onto the doubly-stochastic matrices with
  Sinkhorn-Knopp iterations, which keeps the residual path norm-preserving however deep the stack is

  ``s'_i = post[i] * f(x) + sum_j res[i, j] * s_j``

The maps come from one linear layer on the RMS-normalised, flattened streams (``mapping_proj``: ``n C -> 2 n + n^2``),
three learnable scales (``alpha_pre``, ``alpha_post``, ``alpha_res``) and a bias.  ``pre`` uses a sigmoid, ``post``
twice a sigmoid (so its initial value can be 1), ``res`` a row softmax followed by the Sinkhorn iterations.

Checkpoint keys (reference ``src/mcore_bridge/bridge/gpt_bridge.py:1653-1673``): ``hc_{attn,ffn}_fn`` (the projection),
``hc_{attn,ffn}_base`` (the bias), ``hc_{attn,ffn}_scale`` (the three scales); the block's output contraction uses
``hc_head_{fn,base,scale}``.  The reference takes the module itself from Megatron-Core
(``src/mcore_bridge/model/modules/transformer_block.py:360-365,476-492``), so the arithmetic here follows the published
description of the method; the tests check its invariants (doubly-stochastic ``res``, exact single-stream behaviour at
the identity setting, gradients) rather than a numerical oracle.
"""
from __future__ import annotations

import torch
from torch import nn

from .norm import mark_sequence_parallel


def sinkhorn(m: torch.Tensor, iters: int, eps: float = 1e-6) -> torch.Tensor:
    """Alternating row / column normalisation of positive matrices ``[..., n, n]``."""
    for _ in range(iters):
        m = m / (m.sum(dim=-1, keepdim=True) + eps)
        m = m / (m.sum(dim=-2, keepdim=True) + eps)
    return m


def input_expand(x: torch.Tensor, n: int) -> torch.Tensor:
    """``[T, C]`` -> ``[T, n * C]``: every stream starts as a copy of the embedding."""
    return x.repeat(1, n)


class HyperConnection(nn.Module):

    def __init__(self, config, kind: str = 'layer'):
        super().__init__()
        self.n = n = config.num_residual_streams
        self.c = config.hidden_size
        self.eps = config.layernorm_epsilon
        self.iters = config.mhc_sinkhorn_iterations
        self.kind = kind
        out = n if kind == 'head' else 2 * n + n * n
        dt = config.params_dtype
        self.mapping_proj = nn.Linear(n * self.c, out, bias=False, dtype=torch.float32)
        self.bias = nn.Parameter(torch.zeros(out, dtype=torch.float32))
        g = config.mhc_init_gating_factor
        self.alpha_pre = nn.Parameter(torch.full((1,), g, dtype=torch.float32))
        if kind != 'head':
            self.alpha_post = nn.Parameter(torch.full((1,), g, dtype=torch.float32))
            self.alpha_res = nn.Parameter(torch.full((1,), g, dtype=torch.float32))
        with torch.no_grad():
            self.mapping_proj.weight.zero_()
            if kind != 'head':
                # identity setting: read the mean of the streams, write the output to every stream with weight 1,
                # keep every stream as it is (res = identity after the softmax sharpens the diagonal)
                self.bias[n:2 * n] = 0.0                                   # 2 * sigmoid(0) = 1
                self.bias[2 * n:] = (torch.eye(n) * 8.0).flatten()
        for p in self.parameters():
            mark_sequence_parallel(p, config)       # replicated over TP, sees only this rank's tokens under SP
        del dt

    def _mixes(self, streams: torch.Tensor) -> torch.Tensor:
        x = streams.float()
        rs = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
        return torch.nn.functional.linear(x, self.mapping_proj.weight) * rs

    def pre(self, streams: torch.Tensor):
        """``streams [T, n C]`` -> (sub-layer input ``[T, C]``, ``post [T, n]``, ``res [T, n, n]``)."""
        n, c = self.n, self.c
        mix = self._mixes(streams)
        pre = torch.sigmoid(mix[:, :n] * self.alpha_pre + self.bias[:n])
        post = 2.0 * torch.sigmoid(mix[:, n:2 * n] * self.alpha_post + self.bias[n:2 * n])
        res = torch.softmax((mix[:, 2 * n:] * self.alpha_res + self.bias[2 * n:]).view(-1, n, n), dim=-1)
        res = sinkhorn(res, self.iters)
        pre = pre / pre.sum(-1, keepdim=True).clamp_min(1e-6)
        s = streams.view(-1, n, c)
        x = (pre.unsqueeze(-1) * s.float()).sum(1).to(streams.dtype)
        return x, post, res

    def post(self, out: torch.Tensor, streams: torch.Tensor, post: torch.Tensor, res: torch.Tensor) -> torch.Tensor:
        n, c = self.n, self.c
        s = streams.view(-1, n, c).float()
        new = post.unsqueeze(-1) * out.float().unsqueeze(1) + torch.einsum('tij,tjc->tic', res, s)
        return new.reshape(-1, n * c).to(streams.dtype)

    def contract(self, streams: torch.Tensor) -> torch.Tensor:
        """Output contraction of the block (``kind='head'``): a learned convex combination of the streams."""
        n, c = self.n, self.c
        w = torch.sigmoid(self._mixes(streams) * self.alpha_pre + self.bias)
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-6)
        return (w.unsqueeze(-1) * streams.view(-1, n, c).float()).sum(1).to(streams.dtype)
