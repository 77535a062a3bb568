"""The decoder stack owned by one pipeline stage: layers, activation recomputation, final norm.

Recompute (``recompute_granularity='full'``): ``uniform`` checkpoints every group of
``recompute_num_layers`` layers, ``block`` checkpoints only the first ``recompute_num_layers`` layers of the
stage — the two methods the reference implements in
``src/mcore_bridge/model/modules/transformer_block.py:75-248``.  ``extract_layer_indices`` taps hidden
states after chosen layers (``:326-334,472-474``).
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from ..layers.context import ForwardContext
from ..layers.norm import Norm
from ..parallel import state as ps
from .transformer_layer import TransformerLayer


def get_num_layers_to_build(config, vp_stage: Optional[int] = None) -> int:
    pp = ps.get_pipeline_model_parallel_world_size()
    vpp = config.virtual_pipeline_model_parallel_size or 1
    n = config.num_layers
    first, last = config.num_layers_in_first_pipeline_stage, config.num_layers_in_last_pipeline_stage
    if first is not None or last is not None:
        rank = ps.get_pipeline_model_parallel_rank()
        middle = pp - (first is not None) - (last is not None)
        rest = n - (first or 0) - (last or 0)
        if rank == 0 and first is not None:
            per = first
        elif rank == pp - 1 and last is not None:
            per = last
        else:
            assert middle > 0 and rest % middle == 0
            per = rest // middle
        assert per % vpp == 0
        return per // vpp
    extra = int(config.account_for_embedding_in_pipeline_split) + int(config.account_for_loss_in_pipeline_split)
    total = n + extra
    assert total % (pp * vpp) == 0, f'{total} layers not divisible by pp*vpp = {pp * vpp}'
    per = total // (pp * vpp)
    rank = ps.get_pipeline_model_parallel_rank()
    if config.account_for_embedding_in_pipeline_split and rank == 0 and (vp_stage in (None, 0)):
        per -= 1
    if config.account_for_loss_in_pipeline_split and rank == pp - 1 and (vp_stage in (None, vpp - 1)):
        per -= 1
    return per


def get_transformer_layer_offset(config, vp_stage: Optional[int] = None) -> int:
    """Global index of the first layer this (virtual) stage owns."""
    pp = ps.get_pipeline_model_parallel_world_size()
    rank = ps.get_pipeline_model_parallel_rank()
    vpp = config.virtual_pipeline_model_parallel_size or 1
    vp = vp_stage or 0
    first, last = config.num_layers_in_first_pipeline_stage, config.num_layers_in_last_pipeline_stage
    n = config.num_layers
    if first is not None or last is not None:
        middle = pp - (first is not None) - (last is not None)
        rest = n - (first or 0) - (last or 0)
        per_mid = rest // middle if middle > 0 else 0
        sizes = [(first if (r == 0 and first is not None) else last if (r == pp - 1 and last is not None) else per_mid)
                 for r in range(pp)]
        per_v = [s // vpp for s in sizes]
        return sum(per_v) * vp + sum(per_v[:rank])
    extra_e = int(config.account_for_embedding_in_pipeline_split)
    total = n + extra_e + int(config.account_for_loss_in_pipeline_split)
    per = total // (pp * vpp)
    off = vp * (total // vpp) + rank * per
    if extra_e and not (rank == 0 and vp == 0):
        off -= 1
    return off


class TransformerBlock(nn.Module):
    layer_cls = TransformerLayer          # families with their own decoder layer replace this

    def __init__(self, config, pre_process: bool = True, post_process: bool = True, vp_stage: Optional[int] = None):
        super().__init__()
        self.config = config
        self.pre_process, self.post_process, self.vp_stage = pre_process, post_process, vp_stage
        n = get_num_layers_to_build(config, vp_stage)
        self.layer_offset = get_transformer_layer_offset(config, vp_stage)
        self.layers = nn.ModuleList([self.layer_cls(config, self.layer_offset + i + 1) for i in range(n)])
        self.final_layernorm = Norm(config, config.hidden_size) if post_process else None
        self.input_tensor = None
        # hyper-connections: the streams are contracted where the final norm lives (the last stage); earlier stages
        # pass all n streams on (the activation sent to the next stage is n x as wide)
        self.hc_head = None
        if config.enable_hyper_connections and post_process:
            from ..layers.hyper_connection import HyperConnection
            self.hc_head = HyperConnection(config, kind='head')

    def set_input_tensor(self, t):
        self.input_tensor = t

    def _after_layer(self, h: torch.Tensor, ctx: ForwardContext, index: int) -> torch.Tensor:
        """Deepstack (Qwen3-VL): intermediate vision features are added to the media-token rows after each of the
        first ``L`` decoder layers.  ``ctx.extra['deepstack_visual_embeds']`` is ``[L, n_media_local, H]`` and
        ``ctx.extra['visual_pos_masks']`` ``[T_local]`` (already restricted to this rank's tokens); a text-only
        batch passes no mask and contributes a zero-valued term so the tower still receives gradients.  Parity:
        reference ``src/mcore_bridge/model/mm_gpts/qwen3_vl.py:14-47``."""
        ds = ctx.extra.get('deepstack_visual_embeds')
        if ds is None:
            return h
        layer_index = self.layer_offset + index
        if layer_index >= ds.shape[0]:
            return h
        mask = ctx.extra.get('visual_pos_masks')
        if mask is None:
            return h + ds[layer_index].mean().to(h.dtype) * 0
        rows = mask.reshape(-1).nonzero(as_tuple=True)[0].to(h.device)
        return h.index_add(0, rows, ds[layer_index].to(device=h.device, dtype=h.dtype))

    def _offload_context(self):
        """``cpu_offloading``: the tensors the first ``cpu_offloading_num_layers`` layers save for backward are
        moved to pinned host memory and brought back when their backward runs (parity: the offload hooks of
        reference ``src/mcore_bridge/model/modules/transformer_block.py:468-470``).  Layers under full recompute
        save only their input, so offloading applies to the layers that keep their activations."""
        import contextlib
        cfg = self.config
        if not (cfg.cpu_offloading and self.training and torch.is_grad_enabled()):
            return lambda i: contextlib.nullcontext()
        n_off = cfg.cpu_offloading_num_layers if cfg.cpu_offloading_num_layers is not None else len(self.layers)
        pin = torch.cuda.is_available()

        def ctx_for(i):
            if i < n_off:
                return torch.autograd.graph.save_on_cpu(pin_memory=pin)
            return contextlib.nullcontext()
        return ctx_for

    def _run(self, start: int, end: int):
        def fn(h, ctx):
            for i in range(start, end):
                h = self._after_layer(self.layers[i](h, ctx), ctx, i)
            return h
        return fn

    def forward(self, hidden: Optional[torch.Tensor], ctx: ForwardContext):
        cfg = self.config
        if not self.pre_process:
            hidden = self.input_tensor  # activation received from the previous pipeline stage
        elif cfg.enable_hyper_connections:
            from ..layers.hyper_connection import input_expand
            hidden = input_expand(hidden, cfg.num_residual_streams)      # [T, C] -> [T, n * C]
        offload = self._offload_context()
        taps: List[torch.Tensor] = []
        want = set(cfg.extract_layer_indices or [])
        n = len(self.layers)
        full = cfg.recompute_granularity == 'full' and self.training
        i = 0
        while i < n:
            if full and cfg.recompute_method == 'uniform':
                step = max(1, cfg.recompute_num_layers or 1)
                j = min(n, i + step)
                hidden = checkpoint(self._run(i, j), hidden, ctx, use_reentrant=False)
            elif full and cfg.recompute_method == 'block' and i < (cfg.recompute_num_layers or 0):
                j = i + 1
                hidden = checkpoint(self._run(i, j), hidden, ctx, use_reentrant=False)
            elif full and cfg.recompute_method is None:
                j = i + 1
                hidden = checkpoint(self._run(i, j), hidden, ctx, use_reentrant=False)
            else:
                j = i + 1
                with offload(i):
                    hidden = self._after_layer(self.layers[i](hidden, ctx), ctx, i)
            for g in range(i, j):
                if (self.layer_offset + g) in want:
                    taps.append(hidden)
            i = j
        if self.hc_head is not None:
            ctx.extra['mhc_multistream'] = hidden                        # the MTP layers read the uncontracted streams
            hidden = self.hc_head.contract(hidden)
        if self.final_layernorm is not None:
            hidden = self.final_layernorm(hidden)
        if want:
            return hidden, taps
        return hidden
