"""Lightning attention (linear attention with a fixed per-head decay) of the Ling / Ring hybrid models.

``o_t = scale * S_t^T q_t`` with ``S_t = exp(-slope_h * f_layer) S_{t-1} + k_t v_t^T``; the slopes follow the ALiBi
construction and fade with depth.  Output path: group RMSNorm over the full projection width (statistics reduced
over TP), sigmoid gate from ``g_proj``, row-parallel output projection.  Parameter names as the bridge addresses
them: ``linear_qkv``, ``q_layernorm`` / ``k_layernorm``, ``g_proj``, ``g_norm``, ``linear_proj``.
Parity: reference ``src/mcore_bridge/model/gpts/bailing_hybrid.py:69-229``.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops import gdn as G
from ..ops.rope import qkv_split_norm_rope
from ..parallel import state as ps
from .context import ForwardContext
from .linear import ColumnParallelLinear, RowParallelLinear, _set_tp_attrs
from .norm import Norm


def build_slopes(n_heads: int) -> torch.Tensor:
    """ALiBi-style geometric slopes; for head counts that are not a power of two the closest power of two is used
    and interleaved with the next one's odd entries."""

    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]

    def slopes(n):
        if math.log2(n).is_integer():
            return pow2(n)
        c = 2 ** math.floor(math.log2(n))
        return pow2(c) + slopes(2 * c)[0::2][:n - c]

    return torch.tensor(slopes(n_heads), dtype=torch.float32)


class GroupRMSNorm(nn.Module):
    """RMSNorm applied independently to ``groups`` equal slices of the channel dimension; with TP each rank holds
    whole groups (the weight is sharded like the heads)."""

    def __init__(self, config, hidden: int, groups: int, eps: float):
        super().__init__()
        tp = ps.get_world_size('tp')
        assert groups % tp == 0 and hidden % groups == 0, 'group norm groups must divide over TP'
        self.groups_local, self.width = groups // tp, hidden // groups
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden // tp, dtype=config.params_dtype))
        _set_tp_attrs(self.weight, tp > 1, 0)

    def forward(self, x):
        xf = x.float().view(*x.shape[:-1], self.groups_local, self.width)
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * y.to(x.dtype).view(x.shape)


class LightningAttention(nn.Module):

    def __init__(self, config, layer_number: int):
        super().__init__()
        self.config = config
        tp = ps.get_world_size('tp')
        self.d = config.kv_channels
        self.nq, self.ng = config.num_attention_heads, config.num_query_groups
        assert self.nq % tp == 0 and self.ng % tp == 0
        self.nq_local, self.ng_local, self.qpg = self.nq // tp, self.ng // tp, self.nq // self.ng
        proj = self.nq * self.d
        self.linear_qkv = ColumnParallelLinear(config.hidden_size, (self.nq + 2 * self.ng) * self.d, config,
                                               bias=config.add_qkv_bias)
        if config.qk_layernorm:
            self.q_layernorm = Norm(config, self.d, sequence_parallel_grad=False)
            self.k_layernorm = Norm(config, self.d, sequence_parallel_grad=False)
            for p_ in (self.q_layernorm.weight, self.k_layernorm.weight):     # partial gradient per TP rank
                p_.sequence_parallel = tp > 1
        else:
            self.q_layernorm = self.k_layernorm = None
        self.g_proj = ColumnParallelLinear(config.hidden_size, proj, config, bias=False)
        groups = getattr(config.hf_config, 'group_norm_size', None) or self.nq
        self.g_norm = GroupRMSNorm(config, proj, groups, config.layernorm_epsilon)
        self.linear_proj = RowParallelLinear(proj, config.hidden_size, config, bias=config.add_bias_linear)
        depth = 1 - (layer_number - 1) / max(config.num_layers - 1, 1) + 1e-5
        slope = -build_slopes(self.nq) * depth
        r = ps.get_rank_in('tp') if tp > 1 else 0
        self.register_buffer('slope', slope[r * self.nq_local:(r + 1) * self.nq_local].contiguous(), persistent=False)
        self.use_rope = config.position_embedding_type in ('rope', 'mrope')

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        cfg = self.config
        if ps.get_world_size('cp') > 1:
            raise NotImplementedError('lightning attention does not support context parallelism')
        qkv = self.linear_qkv(x)
        cos, sin = (ctx.cos, ctx.sin) if self.use_rope else (None, None)
        wq = self.q_layernorm.weight if self.q_layernorm is not None else None
        wk = self.k_layernorm.weight if self.k_layernorm is not None else None
        q, k, v, _ = qkv_split_norm_rope(qkv, wq, wk, cos, sin, self.ng_local, self.qpg, self.d, False,
                                         cfg.rotary_interleaved, cfg.layernorm_epsilon,
                                         cfg.layernorm_zero_centered_gamma)
        if self.qpg > 1:
            k = k.repeat_interleave(self.qpg, dim=1)
            v = v.repeat_interleave(self.qpg, dim=1)
        o = G.simple_gla(q.contiguous(), k.contiguous(), v.contiguous(), self.slope, ctx.cu_seqlens)
        o = self.g_norm(o.reshape(o.shape[0], -1))
        gate = self.g_proj(x if not (cfg.sequence_parallel and ps.get_world_size('tp') > 1) else x)
        o = o * torch.sigmoid(gate.float()).to(o.dtype)
        return self.linear_proj(o)
