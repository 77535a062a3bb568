"""Self-attention block: fused-norm QKV projection, per-head q/k norm + rope, core attention, output projection.

Covers standard GQA attention and the gated variant (``attention_output_gate``: the query projection is
doubled, every query head is followed by a gate head and the attention output is multiplied by
``sigmoid(gate)`` — reference ``src/mcore_bridge/model/modules/gated_self_attention.py:55-83``).
Parameter names: ``linear_qkv.{weight,bias,layer_norm_weight}``, ``q_layernorm.weight``,
``k_layernorm.weight``, ``linear_proj.weight`` and, for learnable softmax sinks, ``core_attention.softmax_offset``.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..ops.attention import attention
from ..ops.rope import qkv_split_norm_rope
from ..parallel import state as ps
from ..utils.profiling import nvtx_range
from .context import ForwardContext, layer_cp_comm_type
from .linear import ColumnParallelLinear, LayerNormColumnParallelLinear, RowParallelLinear
from .norm import Norm


class CoreAttention(nn.Module):

    def __init__(self, config, layer_number: int, num_heads_local: int, window=None, scale: Optional[float] = None):
        super().__init__()
        self.config = config
        self.window = window
        self.scale = scale
        self.cp_comm_type = layer_cp_comm_type(config, layer_number)
        if config.softmax_type == 'learnable':
            self.softmax_offset = nn.Parameter(torch.zeros(num_heads_local, dtype=config.params_dtype))
            self.softmax_offset.tensor_model_parallel = ps.get_world_size('tp') > 1
            self.softmax_offset.partition_dim = 0
        else:
            self.register_parameter('softmax_offset', None)
        self.off_by_one = config.softmax_type == 'off-by-one'

    def forward(self, q, k, v, ctx: ForwardContext):
        sinks = self.softmax_offset
        if self.off_by_one:
            sinks = torch.zeros(q.shape[1], device=q.device, dtype=torch.float32)
        cp = ps.get_world_size('cp')
        if cp > 1:
            from ..parallel.context_parallel import cp_attention as ring_attention
            return ring_attention(q, k, v, ctx, scale=self.scale, window=self.window, sinks=sinks,
                                  comm_type=self.cp_comm_type)
        return attention(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, causal=True, scale=self.scale, window=self.window,
                         sinks=sinks, seq_start=ctx.seq_start)


class _ShardedChannelNorm(nn.Module):
    """RMSNorm over ``full`` channels of which this TP rank holds ``local`` (whole heads): the mean square is summed
    over the TP group in forward and backward, the weight shard scales the local channels.  Equivalent to
    gathering the heads, normalising and re-scattering (reference ``src/mcore_bridge/model/gpts/olmoe.py:55-72``)
    at a fraction of the traffic (one float per token instead of the activations)."""

    def __init__(self, config, local: int, full: int):
        super().__init__()
        from .linear import _set_tp_attrs
        self.eps, self.full = config.layernorm_epsilon, full
        self.weight = nn.Parameter(torch.ones(local, dtype=config.params_dtype))
        _set_tp_attrs(self.weight, local != full, 0)

    def forward(self, x):                      # [T, heads_local, d]
        from ..parallel import mappings as M
        xf = x.float()
        ss = M.all_reduce_both(xf.pow(2).sum(dim=(-1, -2)), 'tp')
        inv = torch.rsqrt(ss / self.full + self.eps)
        y = xf * inv[:, None, None] * self.weight.float().view(x.shape[1], x.shape[2])
        return y.to(x.dtype)


class SelfAttention(nn.Module):

    def __init__(self, config, layer_number: int, fuse_input_norm: bool = True, use_rope: bool = True,
                 window=None, rope_key: Optional[str] = None, kv_channels: Optional[int] = None,
                 num_query_groups: Optional[int] = None):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        tp = ps.get_world_size('tp')
        self.d = kv_channels or config.kv_channels
        self.nq = config.num_attention_heads
        self.ng = num_query_groups or config.num_query_groups
        assert self.nq % tp == 0
        # More TP ranks than KV heads: the packed QKV matrix is still split evenly by rows, so a rank's slice cuts
        # through a group [q heads | k | v].  At run time the projection output is all-gathered on the last dim, the
        # rank takes its group and, inside it, its share of the query heads; every `kv_rep` ranks share one KV head
        # (reference ``src/mcore_bridge/model/modules/gated_self_attention.py:23-38,66-72``).
        self.kv_rep = 1
        if self.ng % tp != 0:
            if tp % self.ng != 0:
                raise NotImplementedError(f'TP ({tp}) must divide or be a multiple of num_query_groups ({self.ng})')
            self.kv_rep = tp // self.ng
        self.nq_local, self.ng_local = self.nq // tp, max(1, self.ng // tp)
        self.qpg = self.nq // self.ng
        self.gate = bool(config.attention_output_gate)
        qkv_out = (self.nq * (2 if self.gate else 1) + 2 * self.ng) * self.d
        cls = LayerNormColumnParallelLinear if fuse_input_norm else ColumnParallelLinear
        self.linear_qkv = cls(config.hidden_size, qkv_out, config, bias=config.add_qkv_bias or config.add_bias_linear)
        self.q_norm = self.k_norm = None
        if config.qk_layernorm and config.qk_layernorm_full:
            # one RMSNorm over all heads' channels; the weight is sharded by head, the mean square is reduced over TP
            self.q_layernorm = self.k_layernorm = None
            self.q_norm = _ShardedChannelNorm(config, self.nq_local * self.d, self.nq * self.d)
            self.k_norm = _ShardedChannelNorm(config, self.ng_local * self.d, self.ng * self.d)
        elif config.qk_layernorm:
            self.q_layernorm = Norm(config, self.d, sequence_parallel_grad=False)
            self.k_layernorm = Norm(config, self.d, sequence_parallel_grad=False)
            # replicated weights applied to this rank's heads only: every rank holds a partial gradient, summed over
            # the TP group by the optimizer (the flag it looks at is `sequence_parallel`), with or without SP
            for p_ in (self.q_layernorm.weight, self.k_layernorm.weight):
                p_.sequence_parallel = ps.get_world_size('tp') > 1
        else:
            self.q_layernorm = self.k_layernorm = None
        self.qk_l2_norm = bool(config.qk_l2_norm)
        scale = config.softmax_scale
        self.core_attention = CoreAttention(config, layer_number, self.nq_local, window=window, scale=scale)
        self.linear_proj = RowParallelLinear(self.nq * self.d, config.hidden_size, config, bias=config.add_bias_linear)
        self.use_rope = use_rope and config.position_embedding_type in ('rope', 'mrope')
        self.rope_key = rope_key

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        cfg = self.config
        with nvtx_range('qkv'):
            qkv = self.linear_qkv(x)                              # [T, local packed qkv]
        qpg = self.qpg
        if self.kv_rep > 1:
            from ..parallel import mappings as M
            full = M.all_gather_last_dim_sum_grad(qkv, 'tp')      # [T, ng * group]
            r = ps.get_rank_in('tp')
            mult = 2 if self.gate else 1
            gsize = (self.qpg * mult + 2) * self.d
            grp = full[:, (r // self.kv_rep) * gsize:(r // self.kv_rep + 1) * gsize]
            qpg = self.qpg // self.kv_rep                         # query heads of the group handled here
            q0 = (r % self.kv_rep) * qpg * mult * self.d
            qkv = torch.cat([grp[:, q0:q0 + qpg * mult * self.d], grp[:, self.qpg * mult * self.d:]], dim=-1)
        cos = sin = None
        if self.use_rope:
            if self.rope_key is not None and self.rope_key in ctx.rope_tables:
                cos, sin = ctx.rope_tables[self.rope_key]
            else:
                cos, sin = ctx.cos, ctx.sin
        wq = self.q_layernorm.weight if self.q_layernorm is not None else None
        wk = self.k_layernorm.weight if self.k_layernorm is not None else None
        if self.q_norm is not None:
            q, k, v, gate = qkv_split_norm_rope(qkv, None, None, None, None, self.ng_local, qpg, self.d,
                                                self.gate, cfg.rotary_interleaved, cfg.layernorm_epsilon, False)
            q, k = self.q_norm(q), self.k_norm(k)
            if cos is not None:
                from ..ops.rope import apply_rope
                q, k = apply_rope(q, cos, sin, cfg.rotary_interleaved), apply_rope(k, cos, sin, cfg.rotary_interleaved)
        else:
            q, k, v, gate = qkv_split_norm_rope(qkv, wq, wk, cos, sin, self.ng_local, qpg, self.d, self.gate,
                                                cfg.rotary_interleaved, cfg.layernorm_epsilon,
                                                cfg.layernorm_zero_centered_gamma)
        if self.qk_l2_norm and self.use_rope:
            # Llama-4: weight-less RMS normalisation of q and k after the rotation, on the layers that rotate
            # (``Llama4TextL2Norm`` divides by the root *mean* square)
            def unit_rms(t):
                tf_ = t.float()
                return (tf_ * torch.rsqrt(tf_.pow(2).mean(-1, keepdim=True) + cfg.layernorm_epsilon)).to(t.dtype)
            q, k = unit_rms(q), unit_rms(k)
        with nvtx_range('core_attention'):
            o = self.core_attention(q, k, v, ctx)                 # [T, nq_local, d]
        o = o.reshape(o.shape[0], -1)
        if gate is not None:
            o = o * torch.sigmoid(gate.reshape(o.shape[0], -1).float()).to(o.dtype)
        with nvtx_range('linear_proj'):
            return self.linear_proj(o)
