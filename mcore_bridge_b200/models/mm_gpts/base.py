"""Vision/audio towers that stay Hugging Face modules.

The language model is rebuilt natively; towers are small next to it and change with every model release, so they are
instantiated from the HF config, replicated over TP, and their parameters are copied key-for-key by the bridge
(``module_mapping``: HF prefix -> attribute of the tower wrapper).  A tower's job at run time is
``get_inputs_embeds``: take the text embeddings ``[b, s, H]`` of the *full* (pre-CP, pre-SP) token stream and write
the encoded media into the placeholder positions.  Parity: reference ``src/mcore_bridge/model/mm_gpts/utils.py:27-141``.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
from torch import nn

from ...parallel import state as ps
from ...utils.megatron_utils import split_cp_inputs


def set_config_dtype(hf_config, dtype) -> None:
    """Sets every ``dtype``-like field of a (nested) HF config."""
    from transformers import PretrainedConfig
    for key, value in list(vars(hf_config).items()):
        if isinstance(value, PretrainedConfig):
            set_config_dtype(value, dtype)
        elif key in ('torch_dtype', 'params_dtype', 'dtype'):
            setattr(hf_config, key, dtype)


def vision_config_of(hf_config):
    for k in ('vision_config', 'vit_config'):
        if hasattr(hf_config, k):
            return getattr(hf_config, k)
    return None


def scatter_embeds(inputs_embeds: torch.Tensor, input_ids: torch.Tensor, token_id: int,
                   media_embeds: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Writes ``media_embeds [n, H]`` into the rows where ``input_ids == token_id``; returns (embeds, mask)."""
    mask = input_ids == token_id
    if media_embeds is None:
        return inputs_embeds, mask
    flat = inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
    idx = mask.reshape(-1).nonzero(as_tuple=True)[0]
    if idx.numel() != media_embeds.shape[0]:
        raise ValueError(f'{idx.numel()} placeholder tokens (id {token_id}) but {media_embeds.shape[0]} media '
                         'embeddings')
    flat = flat.index_copy(0, idx, media_embeds.to(flat.dtype).to(flat.device))
    return flat.view_as(inputs_embeds), mask


def local_token_index(total: int, cu_seqlens, config, device) -> torch.Tensor:
    """Indices (into the full token stream of ``total`` tokens) of the tokens this rank's decoder layers see:
    the zig-zag CP chunks first, then this TP rank's contiguous slice under sequence parallelism."""
    idx = torch.arange(total, device=device)
    if config.context_parallel_size > 1:
        idx = split_cp_inputs(idx, cu_seqlens, 0)
    tp = ps.get_world_size('tp')
    if config.sequence_parallel and tp > 1:
        n = idx.numel() // tp
        r = ps.get_rank_in('tp')
        idx = idx[r * n:(r + 1) * n]
    return idx


def shard_token_aligned(mask_full: torch.Tensor, values: torch.Tensor, cu_seqlens, config):
    """``mask_full [T]`` marks media tokens in the full stream and ``values [L, n_media, H]`` holds per-layer data for
    them in stream order.  Returns ``(local_mask [T_local], local_values [L, n_local, H])`` for this rank's tokens."""
    T = mask_full.numel()
    idx = local_token_index(T, cu_seqlens, config, mask_full.device)
    order = torch.cumsum(mask_full.to(torch.int64), 0) - 1          # rank of each media token among media tokens
    local_mask = mask_full[idx]
    sel = order[idx][local_mask]
    if config.sequence_parallel and ps.get_world_size('tp') > 1:
        # every tensor-parallel rank computed the same ``values`` and now keeps the rows of its token slice: the
        # gradient of the (replicated) tower is the sum of the ranks' row gradients
        from ...parallel import mappings as M
        values = M.copy_to_tensor_model_parallel_region(values, 'tp')
    return local_mask, values[:, sel]


class HuggingFaceVit(nn.Module):
    """Base class of tower wrappers.  Subclasses set ``module_mapping`` and implement ``prepare_model`` /
    ``get_inputs_embeds``; ``_vision_tower`` / ``_aligner`` name sub-module prefixes for freezing and LoRA targeting."""
    module_mapping: Dict[str, str] = {}
    _vision_tower = []
    _aligner = []
    _generator = []
    test_mm_type = 'image'

    def __init__(self, config):
        super().__init__()
        self.config = config
        hf_config = config.hf_config
        set_config_dtype(hf_config, config.params_dtype)
        self.hf_config = hf_config
        self.prepare_attn_impl()
        if config.language_model_only:
            self.prepare_language_model(hf_config)
        else:
            self.prepare_model(hf_config)

    # ---- hooks
    def prepare_model(self, hf_config) -> None:
        raise NotImplementedError

    def prepare_language_model(self, hf_config) -> None:
        pass

    def prepare_attn_impl(self) -> None:
        impl = getattr(self.config, 'vit_attn_impl', None)
        if impl:
            self.hf_config._attn_implementation = impl
            vc = vision_config_of(self.hf_config)
            if vc is not None:
                vc._attn_implementation = impl

    def get_inputs_embeds(self, inputs_embeds: torch.Tensor, **inputs) -> Any:
        raise NotImplementedError

    def get_inputs_embeds_language_model(self, inputs_embeds: torch.Tensor, **inputs) -> Any:
        return inputs_embeds

    # ---- shared recipe for Qwen-style towers (patch tensors + grid_thw, image and video placeholders)
    @staticmethod
    def encode_media(visual: nn.Module, inputs: Dict[str, Any], hf_config):
        """Runs the tower once over images and videos together.  Returns ``(image, video, extras, n_image)`` where
        extras is whatever else the tower returned (deepstack features) or ``None``.  A text-only batch still runs
        the tower on a dummy 16x16 grid so that every data-parallel rank executes the same parameters (gradient
        reduction and ZeRO sharding need identical graphs) — the result is multiplied by zero by the caller."""
        pv, pvv = inputs.get('pixel_values'), inputs.get('pixel_values_videos')
        g_i, g_v = inputs.get('image_grid_thw'), inputs.get('video_grid_thw')
        vc = vision_config_of(hf_config)
        dtype = next(visual.parameters()).dtype
        device = next(visual.parameters()).device
        dummy = pv is None and pvv is None
        if dummy:
            feat = vc.in_channels * vc.temporal_patch_size * vc.patch_size ** 2
            pixels = torch.zeros(256, feat, dtype=dtype, device=device)
            grid = torch.tensor([[1, 16, 16]], device=device)
        else:
            parts = [p for p in (pv, pvv) if p is not None]
            grids = [g for p, g in ((pv, g_i), (pvv, g_v)) if p is not None]
            pixels = torch.cat(parts, 0).to(dtype=dtype, device=device)
            grid = torch.cat(grids, 0).to(device)
        res = visual(pixels, grid_thw=grid)
        extras = None
        if hasattr(res, 'pooler_output'):
            embeds, extras = res.pooler_output, getattr(res, 'deepstack_features', None)
        elif isinstance(res, (tuple, list)):
            embeds, extras = res[0], (res[1] if len(res) > 1 else None)
        else:
            embeds = res
        if dummy:
            return embeds, None, extras, None
        n_image = None
        if pv is not None and pvv is not None:
            merge = vc.spatial_merge_size ** 2
            n_image = int((g_i.prod(dim=-1) // merge).sum())
            return embeds[:n_image], embeds[n_image:], extras, n_image
        if pv is not None:
            return embeds, None, extras, None
        return None, embeds, extras, None

    def merge_media(self, inputs_embeds, inputs, visual, hf_config):
        """Text embeddings with image / video embeddings written into their placeholder tokens."""
        ids = inputs['input_ids']
        dummy = inputs.get('pixel_values') is None and inputs.get('pixel_values_videos') is None
        img, vid, _, _ = self.encode_media(visual, inputs, hf_config)
        if dummy:
            return inputs_embeds + img.mean().to(inputs_embeds.dtype) * 0.0
        if img is not None:
            inputs_embeds, _ = scatter_embeds(inputs_embeds, ids, hf_config.image_token_id, img)
        if vid is not None:
            inputs_embeds, _ = scatter_embeds(inputs_embeds, ids, hf_config.video_token_id, vid)
        return inputs_embeds


class HFProxy:
    """Stand-in ``self`` for methods borrowed from a Hugging Face model class (``get_image_features`` and the like):
    attribute look-ups reach the tower wrapper's sub-modules, ``config`` is the HF config the method expects."""

    def __init__(self, tower: nn.Module, hf_config):
        object.__setattr__(self, '_tower', tower)
        object.__setattr__(self, 'config', hf_config)

    def __getattr__(self, name):
        tower = object.__getattribute__(self, '_tower')
        if name in ('dtype', 'device'):          # properties of the Hugging Face base class: answer from the parameters
            return getattr(next(tower.parameters()), name)
        try:
            return getattr(tower, name)
        except AttributeError:
            cls = getattr(tower, 'model_cls', None)
            if cls is not None and hasattr(cls, name):
                attr = getattr(cls, name)
                if isinstance(attr, property):
                    return attr.fget(self)
                return attr.__get__(self) if callable(attr) else attr
            raise
