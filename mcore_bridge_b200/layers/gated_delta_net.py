"""Gated DeltaNet linear-attention block (Qwen3-Next / Qwen3.5).

Parameters (names as the weight bridge addresses them): ``in_proj`` (fused-norm column-parallel, output laid
out per key-head group ``[q | k | v | z | beta | alpha]``), ``conv1d.weight`` (depthwise, channels per group
``[q | k | v]``), ``A_log``, ``dt_bias``, ``out_norm.weight`` (gated RMSNorm over the value head dim) and
``out_proj`` (row-parallel).  Tensor parallelism shards key-head groups; under context parallelism the sequence
shards are exchanged for head shards with one all-to-all before the scan and one after it, and the per-head
parameters are sliced per CP rank (parity: reference
``src/mcore_bridge/model/modules/gated_delta_net.py:47-89,188-377``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import gdn as G
from ..parallel import mappings as M
from ..parallel import state as ps
from ..utils.profiling import nvtx_range
from .context import ForwardContext
from .linear import LayerNormColumnParallelLinear, RowParallelLinear


class GatedDeltaNet(nn.Module):

    def __init__(self, config, layer_number: int):
        super().__init__()
        self.config = config
        cfg = config
        tp = ps.get_world_size('tp')
        self.nk, self.nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        assert self.nk % tp == 0 and self.nv % self.nk == 0
        self.ratio = self.nv // self.nk
        self.nk_local, self.nv_local = self.nk // tp, self.nv // tp
        self.conv_k = cfg.linear_conv_kernel_dim
        self.group_qkvz = 2 * self.dk + 2 * self.ratio * self.dv
        self.group_all = self.group_qkvz + 2 * self.ratio
        self.group_conv = 2 * self.dk + self.ratio * self.dv
        self.in_proj = LayerNormColumnParallelLinear(cfg.hidden_size, self.nk * self.group_all, cfg, bias=False)
        dt = cfg.params_dtype
        self.conv1d = nn.Conv1d(self.nk_local * self.group_conv, self.nk_local * self.group_conv, self.conv_k,
                                groups=self.nk_local * self.group_conv, padding=self.conv_k - 1, bias=False, dtype=dt)
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nv_local, dtype=torch.float32).uniform_(1, 16)).to(dt))
        self.dt_bias = nn.Parameter(torch.ones(self.nv_local, dtype=dt))
        self.out_norm = nn.Module()
        self.out_norm.weight = nn.Parameter(torch.ones(self.dv, dtype=dt))
        # shared by all heads but applied to this rank's heads (and, under CP, this rank's head slice) only: the
        # partial gradients are summed over the TP group by the optimizer
        self.out_norm.weight.sequence_parallel = tp > 1
        for p in (self.conv1d.weight, self.A_log, self.dt_bias):
            p.tensor_model_parallel = tp > 1
            p.partition_dim = 0
            p.no_weight_decay = True
        self.out_proj = RowParallelLinear(self.nv * self.dv, cfg.hidden_size, cfg, bias=False)
        self.eps = cfg.layernorm_epsilon

    def _cp_slice(self, p: torch.Tensor, per_head: int) -> torch.Tensor:
        """Per-head parameter rows owned by this CP rank after the sequence->head all-to-all."""
        cp = ps.get_world_size('cp')
        if cp == 1:
            return p
        r = ps.get_rank_in('cp')
        n = p.shape[0] // cp
        return p[r * n:(r + 1) * n]

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        cp = ps.get_world_size('cp')
        with nvtx_range('in_proj'):
            proj = self.in_proj(x)                                 # [T, nk_local * group_all]
        cu = ctx.cu_seqlens
        if cp > 1:
            proj = M.all_to_all_cp2hp(proj, 'cp')                  # [T * cp (rank-major), cols / cp]
            from ..utils.megatron_utils import cp_gather_index
            index = cp_gather_index(cu, proj.shape[0], cp).to(proj.device)
            proj = proj.index_select(0, index)                     # original token order
        T = proj.shape[0]
        nk = self.nk_local // cp
        nvh = nk * self.ratio
        g = proj.view(T, nk, self.group_all)
        qkv = g[..., :self.group_conv].reshape(T, nk * self.group_conv)
        z = g[..., self.group_conv:self.group_qkvz].reshape(T, nvh, self.dv)
        b = g[..., self.group_qkvz:self.group_qkvz + self.ratio].reshape(T, nvh)
        a = g[..., self.group_qkvz + self.ratio:].reshape(T, nvh)
        w = self._cp_slice(self.conv1d.weight.squeeze(1), self.group_conv)
        with nvtx_range('conv1d'):
            qkv = G.causal_conv1d_silu(qkv.contiguous(), w, None, cu)
        qkv = qkv.view(T, nk, self.group_conv)
        q = qkv[..., :self.dk]
        k = qkv[..., self.dk:2 * self.dk]
        v = qkv[..., 2 * self.dk:].reshape(T, nvh, self.dv)
        q, k = G.l2norm(q), G.l2norm(k)
        if self.ratio > 1:
            q = q.repeat_interleave(self.ratio, dim=1)
            k = k.repeat_interleave(self.ratio, dim=1)
        A_log, dt_bias = self._cp_slice(self.A_log, 1), self._cp_slice(self.dt_bias, 1)
        with nvtx_range('g_and_beta'):
            gdecay = -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())
            beta = torch.sigmoid(b.float())
        with nvtx_range('gated_delta_rule'):
            o = G.chunk_gated_delta_rule(q.contiguous(), k.contiguous(), v.contiguous(), gdecay, beta, cu)
        with nvtx_range('gated_norm'):
            o = G.gated_rmsnorm(o, z, self.out_norm.weight, self.eps).reshape(T, nvh * self.dv)
        if cp > 1:
            from ..utils.megatron_utils import cp_gather_index
            inv = torch.empty_like(index)
            inv[index] = torch.arange(index.numel(), device=index.device)
            o = o.index_select(0, inv)                              # back to rank-major order
            o = M.all_to_all_hp2cp(o, 'cp')
        with nvtx_range('out_proj'):
            return self.out_proj(o)
