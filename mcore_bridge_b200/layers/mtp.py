"""Multi-token prediction (DeepSeek-V3 style), depth ``mtp_num_layers``.

Depth ``k`` predicts token ``t + k + 1`` from the previous depth's hidden state at ``t`` and the embedding of
token ``t + k``: ``h_k = Layer_k(eh_proj([enorm(emb(ids << k)) ; hnorm(h_{k-1})]))``, logits through the shared
output head, cross entropy against the labels shifted ``k`` more positions.  Shifts respect packed-sequence
boundaries and context-parallel chunking (``roll_tensor``).  The MTP losses reach the parameters through
:class:`MTPLossAutoScaler` without changing the returned language-model loss (reference
``src/mcore_bridge/model/gpt_model.py:456-525``; layer structure ``model/modules/mtp_layer.py:375-407``).
``mtp_shared_weights`` unrolls one layer ``mtp_unroll_steps`` times; ``mtp_decoder_input_detach`` cuts the
gradient into the embedding.
"""
from __future__ import annotations

from typing import Dict

import torch
from torch import nn

from ..parallel import mappings as M
from ..parallel import state as ps
from ..utils.megatron_utils import roll_tensor
from .context import ForwardContext, PackedSeqParams
from .linear import ColumnParallelLinear
from .norm import Norm

_MTP_TRACKER: Dict[int, list] = {}


def get_mtp_losses() -> Dict[int, list]:
    """Per-depth ``[sum, count]`` of the logged MTP losses (the trainer averages and clears)."""
    return _MTP_TRACKER


class MTPLossAutoScaler(torch.autograd.Function):
    main_loss_backward_scale: float = 1.0

    @staticmethod
    def forward(ctx, output, mtp_loss):
        ctx.save_for_backward(mtp_loss)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (mtp_loss,) = ctx.saved_tensors
        return grad_output, torch.ones_like(mtp_loss) * MTPLossAutoScaler.main_loss_backward_scale

    @staticmethod
    def set_loss_scale(scale: float):
        MTPLossAutoScaler.main_loss_backward_scale = float(scale)


class MultiTokenPredictionLayer(nn.Module):

    def __init__(self, config, layer_number: int):
        super().__init__()
        from ..models.transformer_layer import TransformerLayer
        self.config = config
        self.enorm = Norm(config, config.hidden_size)
        self.hnorm = Norm(config, config.hidden_size)
        # kept in bf16 even when the rest of the model trains in fp8 (reference mtp_layer.py:34-61)
        self.eh_proj = ColumnParallelLinear(2 * config.hidden_size, config.hidden_size, config, bias=False)
        self.transformer_layer = TransformerLayer(config, config.num_layers + layer_number, is_mtp_layer=True)
        self.final_layernorm = Norm(config, config.hidden_size)

    def forward(self, emb: torch.Tensor, hidden: torch.Tensor, ctx: ForwardContext, sp: bool) -> torch.Tensor:
        x = torch.cat([self.enorm(emb), self.hnorm(hidden)], dim=-1)
        y = self.eh_proj(x)                                         # [T, H/tp] (sequence gathered inside when SP)
        y = M.gather_from_tensor_model_parallel_region(y, 'tp')     # [T, H]
        if sp:
            y = M.scatter_to_sequence_parallel_region(y, 'tp')
        y = self.transformer_layer(y, ctx)
        return self.final_layernorm(y)


class MultiTokenPredictionBlock(nn.Module):

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([MultiTokenPredictionLayer(config, i + 1) for i in range(config.mtp_num_layers)])

    def forward_with_loss(self, model, hidden, ctx: ForwardContext, input_ids, labels, loss_mask, batch, seq, sp):
        """Adds the MTP losses to the graph of ``hidden`` and returns it."""
        cfg = self.config
        steps = cfg.mtp_unroll_steps or len(self.layers)
        cp_group = ps.get_group('cp') if ps.get_world_size('cp') > 1 else None
        psp = PackedSeqParams(cu_seqlens_q=ctx.cu_seqlens, cu_seqlens_kv=ctx.cu_seqlens)
        ids = input_ids.reshape(1, -1)
        lab = labels.reshape(1, -1).clone()
        mask = (torch.ones_like(lab, dtype=torch.float32) if loss_mask is None else loss_mask.reshape(1, -1).float())
        original_tokens = (mask * (lab != -100)).sum()
        h_prev = hidden
        for k in range(steps):
            layer = self.layers[0] if cfg.mtp_shared_weights else self.layers[k]
            ids, _ = roll_tensor(ids, -1, -1, cp_group, psp)
            lab, _ = roll_tensor(lab, -1, -1, cp_group, psp)
            mask, _ = roll_tensor(mask, -1, -1, cp_group, psp)
            emb = model.embed(ids.reshape(-1), ctx, sp)
            if cfg.mtp_decoder_input_detach:
                emb = emb.detach()
            h_k = layer(emb, h_prev, ctx, sp)
            hk_full = model._gather_for_head(h_k, sp)
            tok_loss = model._lm_loss(hk_full, lab.reshape(-1).clamp(min=0)).reshape(1, -1)
            m = mask * (lab != -100)
            n = m.sum()
            mtp_loss = tok_loss * m
            if self.training:
                s = _MTP_TRACKER.setdefault(k, [0.0, 0])
                s[0] = s[0] + (mtp_loss.sum() / n.clamp(min=1)).detach()
                s[1] += 1
            scale = cfg.mtp_loss_scaling_factor / steps
            if cp_group is not None:
                # the mean is over the tokens of the whole sequences: this rank adds its share of it, times cp because
                # gradients are averaged over the dp x cp group afterwards (as for the main loss)
                n = n.clone()
                torch.distributed.all_reduce(n, group=cp_group)
                scale = scale * ps.get_world_size('cp')
            safe_n = n.clamp(min=1)
            if cfg.calculate_per_token_loss:
                hidden = MTPLossAutoScaler.apply(hidden, scale * mtp_loss * (original_tokens / safe_n))
            else:
                hidden = MTPLossAutoScaler.apply(hidden, scale * mtp_loss / safe_n)
            h_prev = h_k
        return hidden
