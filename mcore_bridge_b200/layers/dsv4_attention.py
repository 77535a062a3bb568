"""DeepSeek-V4 attention block (``experimental_attention_variant='dsv4_hybrid'``), sliding-window layers.

Structure (reference ``src/mcore_bridge/model/gpts/deepseek_v4.py:72-325``, which wraps a core attention that lives in
a Megatron-Core development branch):

* queries: ``linear_q_down_proj`` (hidden -> ``q_lora_rank``), ``q_layernorm``, ``linear_q_up_proj``
  (-> heads x ``kv_channels``), then a weight-free RMS norm over every head;
* one shared key / value head: ``linear_kv_proj`` (hidden -> ``kv_channels``), ``kv_layernorm``; the same vector is
  key and value of every query head;
* rotary embedding on the last ``qk_pos_emb_head_dim`` channels of queries and of the shared head, as rotations of the
  pairs ``(2i, 2i+1)`` that leave the channel order unchanged; because values carry the rotation too, the attention
  output is rotated back by the query's angle before the output projection (``:291-316``);
* output: heads are split into ``o_groups`` groups, each group is projected to ``o_lora_rank`` channels by its own
  slice of ``linear_o_group_proj`` (``wo_a``), and ``linear_proj`` (``wo_b``) maps the concatenation to the hidden size
  (``:318-332``).

Core attention of a layer with compression ratio 0 (``layer_types[i] == 'sliding_attention'``): causal attention over
the last ``csa_window_size`` tokens of the same sequence (the token itself included), one learned sink logit per head
in the softmax denominator (``core_attention.attn_sink``), scale ``kv_channels ** -0.5``.  Layers with a non-zero ratio
add compressed key / value blocks and a block selector whose definition is not part of the reference's source tree;
``ModelConfig`` refuses such configurations.

Tensor parallelism: query heads and output groups are split over the TP group (``o_groups % tp == 0``), the shared
key / value head is replicated.  Under sequence parallelism the two down projections and their norms run on the local
tokens and their (narrow) outputs are all-gathered.
"""
from __future__ import annotations

import torch
from torch import nn

from ..ops.attention import attention
from ..ops.rope import apply_rope_ref
from ..parallel import mappings as M
from ..parallel import state as ps
from .context import ForwardContext, layer_cp_comm_type
from .linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear, _set_tp_attrs
from .norm import Norm


def head_rms_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Weight-free RMS norm over the last dimension, computed in fp32."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)).to(x.dtype)


def rope_tail(x: torch.Tensor, cos, sin, rot: int, inverse: bool = False) -> torch.Tensor:
    """Rotate the pairs ``(2i, 2i+1)`` of the last ``rot`` channels of ``x [T, heads, d]``; channel order is kept."""
    head, tail = x[..., :x.shape[-1] - rot], x[..., x.shape[-1] - rot:]
    tail = apply_rope_ref(tail, cos, -sin if inverse else sin, interleaved=True)
    return torch.cat([head, tail], dim=-1)


class _SinkHolder(nn.Module):
    """Carries ``attn_sink`` under the name the checkpoint mapping uses (``core_attention.attn_sink``)."""

    def __init__(self, heads_local: int, dtype, tp: int):
        super().__init__()
        self.attn_sink = nn.Parameter(torch.zeros(heads_local, dtype=dtype))
        _set_tp_attrs(self.attn_sink, tp > 1, 0)
        self.compressor = None
        self.indexer = None


class DSv4SelfAttention(nn.Module):

    def __init__(self, config, layer_number: int):
        super().__init__()
        cfg = config
        self.config, self.layer_number = cfg, layer_number
        ratios = cfg.csa_compress_ratios or []
        ratio = ratios[layer_number - 1] if layer_number - 1 < len(ratios) else 0
        if ratio:
            raise NotImplementedError(f'layer {layer_number}: compressed attention (ratio {ratio}) is not implemented')
        if cfg.q_lora_rank is None:
            raise ValueError('DeepSeek-V4 attention needs q_lora_rank')
        tp = ps.get_world_size('tp')
        self.nh, self.d, self.rot = cfg.num_attention_heads, cfg.kv_channels, cfg.qk_pos_emb_head_dim
        self.groups, self.o_rank = cfg.o_groups, cfg.o_lora_rank
        if self.nh % tp or self.groups % tp or self.nh % self.groups:
            raise NotImplementedError(f'DeepSeek-V4 attention: heads ({self.nh}) and output groups ({self.groups}) '
                                      f'must be multiples of TP ({tp}), heads a multiple of the groups')
        self.nh_local, self.groups_local = self.nh // tp, self.groups // tp
        self.cp_comm_type = layer_cp_comm_type(cfg, layer_number)
        self.linear_q_down_proj = ReplicatedLinear(cfg.hidden_size, cfg.q_lora_rank, cfg)
        self.q_layernorm = Norm(cfg, cfg.q_lora_rank)
        self.linear_q_up_proj = ColumnParallelLinear(cfg.q_lora_rank, self.nh * self.d, cfg, bias=False,
                                                     sequence_parallel=False)
        self.linear_kv_proj = ReplicatedLinear(cfg.hidden_size, self.d, cfg)
        self.kv_layernorm = Norm(cfg, self.d)
        group_in = self.nh * self.d // self.groups
        self.linear_o_group_proj = nn.Parameter(torch.empty(self.groups_local * self.o_rank, group_in,
                                                            dtype=cfg.params_dtype))
        _set_tp_attrs(self.linear_o_group_proj, tp > 1, 0)
        self.linear_proj = RowParallelLinear(self.groups * self.o_rank, cfg.hidden_size, cfg, bias=False)
        self.core_attention = _SinkHolder(self.nh_local, cfg.params_dtype, tp)
        self.window = (int(cfg.csa_window_size) - 1, 0)
        self.scale = cfg.softmax_scale if cfg.softmax_scale is not None else self.d**-0.5

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        cfg = self.config
        tp = ps.get_world_size('tp')
        sp = cfg.sequence_parallel and tp > 1

        def gather(t):
            # narrow outputs of the replicated projections, local tokens -> all tokens; what consumes them sums the
            # gradient over the TP group itself, so the way back only splits
            return M.gather_from_sequence_parallel_region(t, 'tp', tensor_parallel_output_grad=False) if sp else t

        q_c = gather(self.q_layernorm(self.linear_q_down_proj(x)))            # [T, q_lora]
        kv = gather(self.kv_layernorm(self.linear_kv_proj(x)))                # [T, d]
        if tp > 1:      # the shared head feeds this rank's query heads only: its gradient is a per-rank partial sum
            kv = M.copy_to_tensor_model_parallel_region(kv.contiguous(), 'tp')
        T = q_c.shape[0]
        q = self.linear_q_up_proj(q_c).view(T, self.nh_local, self.d)
        q = head_rms_norm(q, cfg.layernorm_epsilon)
        q = rope_tail(q, ctx.cos, ctx.sin, self.rot)
        kv = rope_tail(kv.view(T, 1, self.d), ctx.cos, ctx.sin, self.rot)
        sinks = self.core_attention.attn_sink
        q, kv = q.contiguous(), kv.contiguous()
        if ps.get_world_size('cp') > 1:
            from ..parallel.context_parallel import cp_attention
            o = cp_attention(q, kv, kv, ctx, scale=self.scale, window=self.window, sinks=sinks,
                             comm_type=self.cp_comm_type)
        else:
            o = attention(q, kv, kv, ctx.cu_seqlens, ctx.max_seqlen, causal=True, scale=self.scale,
                          window=self.window, sinks=sinks, seq_start=ctx.seq_start)
        o = rope_tail(o, ctx.cos, ctx.sin, self.rot, inverse=True)           # values were rotated: undo it
        g = self.groups_local
        og = o.reshape(T, g, -1).transpose(0, 1)                              # [g, T, heads/g * d]
        w = self.linear_o_group_proj.view(g, self.o_rank, -1)
        y = torch.bmm(og, w.transpose(1, 2).to(og.dtype)).transpose(0, 1).reshape(T, g * self.o_rank)
        return self.linear_proj(y)
