"""Multi-latent attention (DeepSeek-V2/V3 style) with the optional DSA lightning indexer (DeepSeek-V3.2 / GLM-5).

Projections (names as the weight bridge addresses them):
``linear_q_proj`` or ``linear_q_down_proj`` -> (``linear_q_up_proj.layer_norm_weight``) -> ``linear_q_up_proj``;
``linear_kv_down_proj`` -> split ``[kv_lora | k_pe]`` -> (``linear_kv_up_proj.layer_norm_weight``) ->
``linear_kv_up_proj``; ``linear_proj``.  The down projections are replicated and run on the local
(sequence-parallel) tokens; their small outputs are all-gathered before the head-sharded up projections
(parity with the gather/scatter fix-ups at reference
``src/mcore_bridge/model/modules/multi_latent_attention.py:43-88``).  Rotary embedding acts on the
``qk_pos_emb_head_dim`` sub-vector as interleaved pairs, ``k_pe`` is shared by all heads (``:139-173``).

DSA (``experimental_attention_variant='dsa'``): an indexer scores every (query, key) pair,
``score[s,t] = sum_h w[s,h] * relu(q_idx[s,h] . k_idx[t])``, keeps the top-k keys per query and attention
runs over those keys only (reference ``src/mcore_bridge/patcher.py:245-380``).  The Hadamard
``rotate_activation`` of the reference is orthogonal and cancels in ``q . k``; it only matters for fp8
quantisation of the indexer operands and is applied there.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops.attention import attention, segment_ids
from ..ops.norm import layernorm_ref
from ..ops.rope import apply_rope_ref
from ..parallel import mappings as M
from ..parallel import state as ps
from .context import ForwardContext
from .linear import ColumnParallelLinear, LayerNormColumnParallelLinear, ReplicatedLinear, RowParallelLinear


def _yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def rope_interleaved_to_half(x: torch.Tensor, cos, sin) -> torch.Tensor:
    """MLA rope: pairs ``(2i, 2i+1)`` are rotated and the result is laid out ``[evens | odds]`` — the same
    output order Transformers' ``apply_rotary_pos_emb_interleave`` produces, so q.k matches bit for bit."""
    d = x.shape[-1]
    x = x.reshape(*x.shape[:-1], d // 2, 2).transpose(-1, -2).reshape(*x.shape[:-1], d)
    return apply_rope_ref(x, cos, sin, interleaved=False)


class DSAIndexer(nn.Module):

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.n_heads = config.dsa_indexer_n_heads
        self.head_dim = config.dsa_indexer_head_dim
        self.topk = config.dsa_indexer_topk
        self.rope_dim = config.qk_pos_emb_head_dim
        self.linear_wq_b = ReplicatedLinear(config.q_lora_rank, self.n_heads * self.head_dim, config,
                                            sequence_parallel_grad=False)
        self.linear_wk = ReplicatedLinear(config.hidden_size, self.head_dim, config, sequence_parallel_grad=False)
        self.k_norm = nn.LayerNorm(self.head_dim, eps=1e-6, dtype=config.params_dtype)
        self.linear_weights_proj = ReplicatedLinear(config.hidden_size, self.n_heads, config,
                                                    sequence_parallel_grad=False)
        self.softmax_scale = self.head_dim**-0.5

    def _rope(self, x, cos, sin):
        pe, nope = x[..., :self.rope_dim], x[..., self.rope_dim:]
        if self.config.dsa_indexer_rotary_interleaved:
            pe = rope_interleaved_to_half(pe, cos, sin)
        else:
            pe = apply_rope_ref(pe, cos, sin, interleaved=False)
        return torch.cat([pe, nope], dim=-1)

    def forward_before_topk(self, x: torch.Tensor, qr: torch.Tensor, ctx: ForwardContext):
        """``x [T, H]``, ``qr [T, q_lora]`` (both already gathered over SP) -> ``q [T, h, d]``, ``k [T, d]``,
        ``w [T, h]``."""
        T = x.shape[0]
        q = self.linear_wq_b(qr).view(T, self.n_heads, self.head_dim)
        q = self._rope(q, ctx.cos, ctx.sin)
        k = self.linear_wk(x)
        k = layernorm_ref(k, self.k_norm.weight, self.k_norm.bias, self.k_norm.eps)
        k = self._rope(k.view(T, 1, self.head_dim), ctx.cos, ctx.sin).view(T, self.head_dim)
        w = self.linear_weights_proj(x).float() * (self.n_heads**-0.5) * self.softmax_scale
        return q, k, w

    def index_scores(self, q, k, w, mask: torch.Tensor) -> torch.Tensor:
        """``[T, T]`` fp32 scores with ``-inf`` where ``mask`` is False."""
        from ..ops import dsa
        return dsa.index_scores(q, k, w, mask)

    def forward(self, x, qr, ctx: ForwardContext, mask: torch.Tensor, gather_keys=None):
        """``gather_keys``: under context parallelism, maps this rank's keys to the keys of the whole stream."""
        from ..ops import dsa
        q, k, w = self.forward_before_topk(x, qr, ctx)
        if gather_keys is not None:
            k = gather_keys(k)
        T = q.shape[0]
        topk = min(self.topk, k.shape[0])
        if mask is None and not (not torch.is_grad_enabled() and dsa.cuda_indexer_supported(q, k)
                                 and ps.get_world_size('cp') == 1):
            seg = segment_ids(ctx.cu_seqlens, T)
            pos = torch.arange(T, device=q.device)
            mask = (seg[:, None] == seg[None, :]) & (pos[None, :] <= pos[:, None])
        if not torch.is_grad_enabled() and dsa.cuda_indexer_supported(q, k) and ps.get_world_size('cp') == 1:
            # selection only (the indexer is not being trained through this call): tcgen05 scores + radix select
            seq_start = ctx.seq_start
            if seq_start is None:
                from ..ops.attention_cuda import seq_start_from_cu
                seq_start = seq_start_from_cu(ctx.cu_seqlens, T, q.device)
            scores = dsa.index_scores_cuda(q, k, w, seq_start)
            return dsa.topk_indices(scores, topk), scores
        scores = self.index_scores(q, k, w, mask)
        idx = scores.topk(topk, dim=-1).indices
        return idx, scores


class MLASelfAttention(nn.Module):

    def __init__(self, config, layer_number: int):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        from .context import layer_cp_comm_type
        self.cp_comm_type = layer_cp_comm_type(config, layer_number)
        cfg = config
        tp = ps.get_world_size('tp')
        self.nh = cfg.num_attention_heads
        assert self.nh % tp == 0
        self.nh_local = self.nh // tp
        self.qk_nope, self.qk_rope, self.v_dim = cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim
        self.q_dim = self.qk_nope + self.qk_rope
        self.kv_lora = cfg.kv_lora_rank
        if cfg.q_lora_rank is None:
            self.linear_q_proj = ColumnParallelLinear(cfg.hidden_size, self.nh * self.q_dim, cfg, bias=False)
        else:
            self.linear_q_down_proj = ReplicatedLinear(cfg.hidden_size, cfg.q_lora_rank, cfg)
            self.linear_q_up_proj = LayerNormColumnParallelLinear(cfg.q_lora_rank, self.nh * self.q_dim, cfg,
                                                                  bias=False, sequence_parallel=False)
            self.linear_q_up_proj.layer_norm_weight.sequence_parallel = False  # sees all tokens, full gradient
        self.linear_kv_down_proj = ReplicatedLinear(cfg.hidden_size, self.kv_lora + self.qk_rope, cfg)
        self.linear_kv_up_proj = LayerNormColumnParallelLinear(self.kv_lora, self.nh * (self.qk_nope + self.v_dim), cfg,
                                                               bias=False, sequence_parallel=False)
        self.linear_kv_up_proj.layer_norm_weight.sequence_parallel = False
        self.linear_proj = RowParallelLinear(self.nh * self.v_dim, cfg.hidden_size, cfg, bias=cfg.add_bias_linear)
        scale = cfg.softmax_scale if cfg.softmax_scale is not None else self.q_dim**-0.5
        rs = cfg.rope_scaling or {}
        if rs.get('rope_type', rs.get('type')) == 'yarn' and rs.get('mscale_all_dim'):
            m = _yarn_mscale(rs['factor'], rs['mscale_all_dim'])
            scale = scale * m * m
        self.scale = scale
        self.indexer = DSAIndexer(cfg) if cfg.experimental_attention_variant == 'dsa' else None
        self.indexer_loss = None

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        cfg = self.config
        sp = cfg.sequence_parallel and ps.get_world_size('tp') > 1
        tp = ps.get_world_size('tp')

        def gather(t):
            # Outputs of the replicated down projections on local tokens -> all tokens.  Their consumers (the
            # column-parallel up projections) all-reduce the input gradient themselves, so the gradient coming
            # back here is already complete and is only split, not summed again.
            return M.gather_from_sequence_parallel_region(t, 'tp', tensor_parallel_output_grad=False) if sp else t

        if cfg.q_lora_rank is None:
            q = self.linear_q_proj(x)                             # column-parallel: gathers the sequence itself
            qr = None
        else:
            q_c = gather(self.linear_q_down_proj(x))              # [T, q_lora]
            self.linear_q_up_proj.return_layernorm_output = True
            q, qr = self.linear_q_up_proj(q_c)
            self.linear_q_up_proj.return_layernorm_output = False
        kv_c = gather(self.linear_kv_down_proj(x))                # [T, kv_lora + rope]
        kv_lat, k_pe = kv_c[:, :self.kv_lora], kv_c[:, self.kv_lora:]
        if tp > 1:  # k_pe feeds every local head: its gradient is a per-rank partial sum
            k_pe = M.copy_to_tensor_model_parallel_region(k_pe.contiguous(), 'tp')
        T = q.shape[0]
        if self.indexer is not None and self._use_gather_path(T):
            return self.linear_proj(self._sparse_attention_absorbed(x, qr, q, kv_lat, k_pe, ctx, sp).reshape(T, -1))
        kv = self.linear_kv_up_proj(kv_lat.contiguous())          # [T, nh_local * (nope + v)]
        q = q.view(T, self.nh_local, self.q_dim)
        kv = kv.view(T, self.nh_local, self.qk_nope + self.v_dim)
        q_nope, q_pe = q[..., :self.qk_nope], q[..., self.qk_nope:]
        k_nope, v = kv[..., :self.qk_nope], kv[..., self.qk_nope:]
        rope = rope_interleaved_to_half if cfg.mla_rope_interleaved else apply_rope_ref
        q_pe = rope(q_pe, ctx.cos, ctx.sin)
        k_pe = rope(k_pe.reshape(T, 1, self.qk_rope), ctx.cos, ctx.sin)
        q = torch.cat([q_nope, q_pe], dim=-1)
        k = torch.cat([k_nope, k_pe.expand(T, self.nh_local, self.qk_rope)], dim=-1)
        v = v.contiguous()
        if self.indexer is not None:
            o = self._sparse_attention(x, qr, q, k, v, ctx, sp)
        elif ps.get_world_size('cp') > 1:
            # this rank holds two zig-zag chunks of every sequence: keys / values are exchanged over the group
            from ..parallel.context_parallel import cp_attention as ring_attention
            o = ring_attention(q.contiguous(), k.contiguous(), v, ctx, scale=self.scale,
                               comm_type=self.cp_comm_type)
        else:
            o = attention(q.contiguous(), k.contiguous(), v, ctx.cu_seqlens, ctx.max_seqlen, causal=True,
                          scale=self.scale)
        return self.linear_proj(o.reshape(T, -1))

    def _use_gather_path(self, T: int) -> bool:
        """Long inputs take the weight-absorbed, gather-based sparse attention (memory ``O(T * topk)``); short ones the
        dense-masked form, which also serves the KL-trained indexer.  ``MCB200_DSA_GATHER_MIN_T`` moves the switch."""
        import os
        cfg = self.config
        if self.training and cfg.dsa_indexer_loss_coeff > 0:
            return False
        if ps.get_world_size('cp') > 1:
            return False
        return T >= int(os.environ.get('MCB200_DSA_GATHER_MIN_T', '4096'))

    def _sparse_attention_absorbed(self, x, qr, q, kv_lat, k_pe, ctx: ForwardContext, sp: bool):
        cfg = self.config
        from ..ops import dsa
        T = q.shape[0]
        up = self.linear_kv_up_proj
        # with a LoRA adapter on this projection the slot holds the wrapper: norm from the wrapped layer, matrix with
        # the adapter's low-rank update added
        weight = up.effective_weight() if hasattr(up, 'effective_weight') else up.weight
        up = getattr(up, 'base_layer', up)
        lat_n = up.norm(kv_lat.contiguous())                                    # normalised latent [T, kv_lora]
        if ps.get_world_size('tp') > 1:       # feeds this rank's heads only: the gradient is a per-rank partial sum
            lat_n = M.copy_to_tensor_model_parallel_region(lat_n, 'tp')
        W = weight.view(self.nh_local, self.qk_nope + self.v_dim, self.kv_lora)
        q = q.view(T, self.nh_local, self.q_dim)
        q_nope, q_pe = q[..., :self.qk_nope], q[..., self.qk_nope:]
        rope = rope_interleaved_to_half if cfg.mla_rope_interleaved else apply_rope_ref
        q_pe = rope(q_pe, ctx.cos, ctx.sin)
        k_pe = rope(k_pe.reshape(T, 1, self.qk_rope), ctx.cos, ctx.sin).reshape(T, self.qk_rope)
        xg = M.gather_from_sequence_parallel_region(x, 'tp', tensor_parallel_output_grad=False) if sp else x
        with torch.no_grad():
            idx, _ = self.indexer(xg.detach(), qr.detach(), ctx, None)
        seq_start = ctx.seq_start
        if seq_start is None:
            seg = segment_ids(ctx.cu_seqlens, T)
            starts = ctx.cu_seqlens[:-1].to(torch.int64) if ctx.cu_seqlens is not None else \
                torch.zeros(1, dtype=torch.int64, device=q.device)
            seq_start = starts.to(q.device)[seg]
        return dsa.sparse_mla_attention_absorbed(q_nope, q_pe, lat_n, k_pe, W[:, :self.qk_nope], W[:, self.qk_nope:],
                                                 idx, seq_start, self.scale)

    def _sparse_attention(self, x, qr, q, k, v, ctx: ForwardContext, sp: bool):
        """Top-k sparse attention.  The indexer runs without gradient for the main loss (as in the Hugging Face
        model); with ``dsa_indexer_loss_coeff > 0`` a KL term trains it towards the attention distribution."""
        cfg = self.config
        T = q.shape[0]
        xg = M.gather_from_sequence_parallel_region(x, 'tp', tensor_parallel_output_grad=False) if sp else x
        gather_keys = None
        if ps.get_world_size('cp') > 1:
            # queries are this rank's zig-zag chunks, keys / values (and the indexer's keys) those of the whole stream
            from ..parallel.context_parallel import gather_to_stream_order, stream_index_of_local_tokens

            def gather_keys(t):
                return gather_to_stream_order(t, ctx)

            k, v = gather_keys(k.contiguous()), gather_keys(v)
            qpos = stream_index_of_local_tokens(ctx, q.device)
            seg = segment_ids(ctx.cu_seqlens, k.shape[0])
            mask = (seg[qpos][:, None] == seg[None, :]) & (torch.arange(k.shape[0], device=q.device)[None, :]
                                                            <= qpos[:, None])
        else:
            seg = segment_ids(ctx.cu_seqlens, T)
            pos = torch.arange(T, device=q.device)
            mask = (seg[:, None] == seg[None, :]) & (pos[None, :] <= pos[:, None])
        train_indexer = self.training and cfg.dsa_indexer_loss_coeff > 0
        with torch.set_grad_enabled(train_indexer):
            idx, scores = self.indexer(xg.detach() if not train_indexer else xg.detach(),
                                       qr.detach(), ctx, mask, gather_keys)
        from ..ops import dsa
        o, attn_probs = dsa.sparse_attention(q, k, v, idx, mask, self.scale, need_probs=train_indexer)
        if train_indexer:
            # the target distribution sums the heads of every tensor-parallel rank; under context parallelism the
            # queries here are this rank's part of the stream and the loss its share of the stream's mean
            loss = dsa.indexer_kl_loss(scores, attn_probs.detach(), mask,
                                       idx if cfg.dsa_indexer_use_sparse_loss else None, head_group='tp',
                                       token_share=ps.get_world_size('cp'))
            from ..ops.moe import MoEAuxLossAutoScaler
            o = MoEAuxLossAutoScaler.apply(o, loss * cfg.dsa_indexer_loss_coeff)
            self.indexer_loss = loss.detach()
        return o
