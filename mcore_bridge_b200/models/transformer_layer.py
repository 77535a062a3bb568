"""One decoder layer: attention variant + residual, then dense MLP or MoE + residual.

Which sub-modules a layer gets is decided by its (1-based) ``layer_number`` and the config patterns:
MoE vs dense (``moe_layer_freq``), gated-DeltaNet vs full attention (``linear_attention_freq``), sliding
window (``window_attn_skip_freq``), rope skipping (``no_rope_freq``), MLA / DSA
(``multi_latent_attention`` / ``experimental_attention_variant``).  Norms are folded into the following
linear where that linear is column-parallel (``linear_qkv.layer_norm_weight``,
``mlp.linear_fc1.layer_norm_weight``); MoE layers and MLA keep stand-alone ``pre_mlp_layernorm`` /
``input_layernorm`` modules — the naming the weight bridge relies on (reference
``src/mcore_bridge/bridge/gpt_bridge.py:1619-1651``).

``mlp_padding_free`` drops padding tokens before the MLP/MoE and restores them afterwards (reference
``src/mcore_bridge/model/modules/transformer_layer.py:343-375``).
"""
from __future__ import annotations


import torch
from torch import nn

from ..layers.attention import SelfAttention
from ..layers.context import ForwardContext
from ..layers.mlp import MLP
from ..layers.moe import MoELayer
from ..layers.norm import Norm
from ..parallel import mappings as M
from ..parallel import state as ps
from ..utils.profiling import nvtx_range


def _identity(x):
    return x


class TransformerLayer(nn.Module):

    def __init__(self, config, layer_number: int, is_mtp_layer: bool = False):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        idx = min(layer_number - 1, config.num_layers - 1)  # MTP layers reuse the last layer's pattern entry
        self.is_moe = bool(config.moe_layer_pattern()[idx]) if config.num_moe_experts else False
        self.is_linear_attention = bool(config.linear_attention_pattern()[idx]) and not is_mtp_layer
        use_rope = not bool(config.no_rope_pattern()[idx])
        window = config.window_size if config.window_pattern()[idx] else None
        variant = config.experimental_attention_variant
        self.input_layernorm = None
        if self.is_linear_attention and variant == 'gated_delta_net':
            from ..layers.gated_delta_net import GatedDeltaNet
            self.self_attention = GatedDeltaNet(config, layer_number)
        elif self.is_linear_attention and variant == 'lightning':
            from ..layers.lightning_attention import LightningAttention
            self.input_layernorm = Norm(config, config.hidden_size)
            self.self_attention = LightningAttention(config, layer_number)
        elif variant == 'dsv4_hybrid':
            from ..layers.dsv4_attention import DSv4SelfAttention
            self.input_layernorm = Norm(config, config.hidden_size)
            self.self_attention = DSv4SelfAttention(config, layer_number)
        elif config.multi_latent_attention:
            from ..layers.mla import MLASelfAttention
            self.input_layernorm = Norm(config, config.hidden_size)
            self.self_attention = MLASelfAttention(config, layer_number)
        else:
            self.self_attention = SelfAttention(config, layer_number, fuse_input_norm=True, use_rope=use_rope,
                                                window=window)
        if self.is_moe:
            self.pre_mlp_layernorm = Norm(config, config.hidden_size)
            self.mlp = MoELayer(config, layer_number)
        else:
            self.pre_mlp_layernorm = None
            self.mlp = MLP(config, fuse_input_norm=True)
        self.self_attention_hyper_connection = self.mlp_hyper_connection = None
        if config.enable_hyper_connections:
            from ..layers.hyper_connection import HyperConnection
            self.self_attention_hyper_connection = HyperConnection(config)
            self.mlp_hyper_connection = HyperConnection(config)
        if config.post_sublayer_layernorm:
            # sandwich norms live on the sub-modules so their names match the checkpoint layout
            self.self_attention.post_self_attn_layernorm = Norm(config, config.hidden_size)
            self.mlp.post_mlp_layernorm = Norm(config, config.hidden_size)

    def _attention(self, hidden, ctx):
        hc = self.self_attention_hyper_connection
        if hc is not None:
            streams = hidden                                 # [T, n * C]: the sub-layer reads a mix of the streams
            hidden, post, res = hc.pre(streams)
        x = hidden if self.input_layernorm is None else self.input_layernorm(hidden)
        with nvtx_range('attention'):
            out = self.self_attention(x, ctx)
        if self.config.post_sublayer_layernorm:
            out = self.self_attention.post_self_attn_layernorm(out)
        if hc is not None:
            return hc.post(out, streams, post, res)
        return hidden + out

    def _mlp(self, hidden, ctx: ForwardContext):
        cfg = self.config
        hc = self.mlp_hyper_connection
        if hc is not None:
            streams = hidden
            hidden, post, res = hc.pre(streams)
        x = hidden if self.pre_mlp_layernorm is None else self.pre_mlp_layernorm(hidden)
        with nvtx_range('moe' if self.is_moe else 'mlp'):
            if self.is_moe:
                out = self.mlp(x, ctx.padding_mask, ctx.seg_ids, ctx.num_seqs, ctx.input_ids)
            else:
                out = self.mlp(x)
        if cfg.post_sublayer_layernorm:
            out = self.mlp.post_mlp_layernorm(out)
        if hc is not None:
            return hc.post(out, streams, post, res)
        return hidden + out

    def _mlp_padding_free(self, hidden, ctx: ForwardContext):
        """Run the MLP on non-padding tokens only.  Under sequence parallelism the tokens are gathered,
        filtered, padded to a multiple of TP and scattered again, and the inverse afterwards."""
        cfg = self.config
        sp = cfg.sequence_parallel and ps.get_world_size('tp') > 1
        x = hidden if self.pre_mlp_layernorm is None else None
        h = hidden
        if sp:
            h = M.gather_from_sequence_parallel_region(h, tensor_parallel_output_grad=False)
        keep = ~ctx.extra['full_padding_mask']
        sel = keep.nonzero(as_tuple=True)[0]
        hs = h.index_select(0, sel)
        pad = 0
        if sp:
            tp = ps.get_world_size('tp')
            pad = (-hs.shape[0]) % tp
            if pad:
                hs = torch.nn.functional.pad(hs, (0, 0, 0, pad))
            hs = M.scatter_to_sequence_parallel_region(hs)
        sub = ForwardContext(**{**ctx.__dict__, 'padding_mask': None, 'seg_ids': None})
        xs = hs if self.pre_mlp_layernorm is None else self.pre_mlp_layernorm(hs)
        out = self.mlp(xs, None, None, None) if self.is_moe else self.mlp(xs)
        if sp:
            out = M.gather_from_sequence_parallel_region(out, tensor_parallel_output_grad=False)
            if pad:
                out = out[:-pad]
        full = torch.zeros_like(h).index_copy(0, sel, out)
        if sp:
            full = M.scatter_to_sequence_parallel_region(full)
        return hidden + full

    def _selective(self, name: str) -> bool:
        """Selective recompute: ``recompute_modules`` names the sub-blocks whose activations are dropped and recomputed
        in backward.  ``mlp`` / ``moe`` cover the feed-forward block (norm included), ``self_attn`` the whole attention
        block; ``core_attn`` needs nothing here because the attention kernels keep only their output and
        log-sum-exp, and ``layernorm`` nothing because the fused norm-linear blocks already recompute the norm
        (reference ``src/mcore_bridge/model/modules/transformer_layer.py:144-196``)."""
        cfg = self.config
        return (self.training and cfg.recompute_granularity == 'selective' and name in (cfg.recompute_modules or ())
                and torch.is_grad_enabled())

    # names of ``offload_modules`` that belong to the attention block and to the feed-forward block
    _ATTN_OFFLOAD = frozenset({'attn_norm', 'qkv_linear', 'core_attn', 'attn_proj', 'self_attn'})
    _MLP_OFFLOAD = frozenset({'mlp_norm', 'mlp', 'moe', 'moe_act', 'expert_fc1', 'expert_fc2', 'shared_expert',
                              'dense_mlp'})

    def _offload(self, names):
        """``fine_grained_activation_offloading``: while a sub-block named in ``offload_modules`` runs, the tensors it
        saves for backward go to (pinned) host memory and come back when its backward runs.  The granularity is the
        sub-block (attention incl. its norm and projections / feed-forward incl. its norm), the finest at which this
        layer keeps activations: the fused norm-linear and gated-activation blocks save one tensor each (reference
        ``src/mcore_bridge/model/modules/transformer_layer.py:197-209``)."""
        import contextlib
        cfg = self.config
        if (cfg.fine_grained_activation_offloading and self.training and torch.is_grad_enabled()
                and names & set(cfg.offload_modules or ())):
            return torch.autograd.graph.save_on_cpu(pin_memory=torch.cuda.is_available())
        return contextlib.nullcontext()

    def forward(self, hidden: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        from torch.utils.checkpoint import checkpoint
        if self._selective('self_attn'):
            hidden = checkpoint(self._attention, hidden, ctx, use_reentrant=False)
        else:
            with self._offload(self._ATTN_OFFLOAD):
                hidden = self._attention(hidden, ctx)
        if self.config.mlp_padding_free and ctx.extra.get('full_padding_mask') is not None:
            return self._mlp_padding_free(hidden, ctx)
        if self._selective('moe' if self.is_moe else 'mlp'):
            return checkpoint(self._mlp, hidden, ctx, use_reentrant=False)
        with self._offload(self._MLP_OFFLOAD):
            return self._mlp(hidden, ctx)
