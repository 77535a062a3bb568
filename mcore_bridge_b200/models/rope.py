"""Rotary position embedding tables: inverse frequencies for every scaling family and per-token cos/sin.

Families: default, linear, dynamic (NTK), yarn, longrope, llama3 and ``dynamic_alpha`` (Hunyuan), the set
the reference obtains from Transformers' ``ROPE_INIT_FUNCTIONS`` (``src/mcore_bridge/model/rope.py:113-192``).
They are computed here directly from the published formulas so the module does not depend on a
Transformers version; ``tests/test_rope.py`` checks them against Transformers.

:class:`RotaryEmbedding` turns position ids into per-token ``cos``/``sin`` of shape ``[T, rot/2]`` (fp32,
attention scaling folded in), including MRoPE (3-axis positions, sectioned or interleaved).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def _rope_type(rope_scaling: Optional[dict]) -> str:
    if not rope_scaling:
        return 'default'
    t = rope_scaling.get('rope_type', rope_scaling.get('type', 'default'))
    if t == 'dynamic' and rope_scaling.get('alpha') is not None:
        t = 'dynamic_alpha'
    if t == 'su':
        t = 'longrope'
    return t


def _base_inv_freq(base: float, dim: int) -> torch.Tensor:
    return 1.0 / (base**(torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))


def _yarn_mscale(scale: float, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def compute_inv_freq(rope_type: str, base: float, dim: int, rope_scaling: Optional[dict],
                     max_position_embeddings: Optional[int], seq_len: Optional[int] = None,
                     original_max_position_embeddings: Optional[int] = None) -> Tuple[torch.Tensor, float]:
    """Returns ``(inv_freq [dim/2], attention_scaling)``."""
    rs = rope_scaling or {}
    if rope_type == 'default':
        return _base_inv_freq(base, dim), 1.0
    if rope_type == 'linear':
        return _base_inv_freq(base, dim) / rs['factor'], 1.0
    if rope_type == 'dynamic':
        factor = rs['factor']
        max_pos = max_position_embeddings
        sl = max(seq_len or 0, max_pos)
        nb = base * ((factor * sl / max_pos) - (factor - 1))**(dim / (dim - 2))
        return _base_inv_freq(nb, dim), 1.0
    if rope_type == 'dynamic_alpha':
        nb = base * rs['alpha']**(dim / (dim - 2))
        return _base_inv_freq(nb, dim), 1.0
    if rope_type == 'yarn':
        factor = rs['factor']
        orig = rs.get('original_max_position_embeddings') or original_max_position_embeddings
        if orig is None:
            orig = max_position_embeddings
        elif rs.get('original_max_position_embeddings') and max_position_embeddings and 'factor' not in rs:
            factor = max_position_embeddings / orig
        attention_factor = rs.get('attention_factor')
        mscale, mscale_all_dim = rs.get('mscale'), rs.get('mscale_all_dim')
        if attention_factor is None:
            if mscale and mscale_all_dim:
                attention_factor = float(_yarn_mscale(factor, mscale) / _yarn_mscale(factor, mscale_all_dim))
            else:
                attention_factor = _yarn_mscale(factor)
        beta_fast, beta_slow = rs.get('beta_fast') or 32, rs.get('beta_slow') or 1

        def corr_dim(num_rot):
            return (dim * math.log(orig / (num_rot * 2 * math.pi))) / (2 * math.log(base))

        low, high = corr_dim(beta_fast), corr_dim(beta_slow)
        if rs.get('truncate', True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, dim - 1)
        pos_freqs = base**(torch.arange(0, dim, 2).float() / dim)
        extrapolation, interpolation = 1.0 / pos_freqs, 1.0 / (factor * pos_freqs)
        if low == high:
            high += 0.001
        ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
        extrap_factor = 1 - ramp
        inv = interpolation * (1 - extrap_factor) + extrapolation * extrap_factor
        return inv, float(attention_factor)
    if rope_type == 'llama3':
        inv = _base_inv_freq(base, dim)
        factor, lo, hi = rs['factor'], rs['low_freq_factor'], rs['high_freq_factor']
        old = rs['original_max_position_embeddings']
        low_wl, high_wl = old / lo, old / hi
        wavelen = 2 * math.pi / inv
        out = torch.where(wavelen > low_wl, inv / factor, inv)
        smooth = (old / wavelen - lo) / (hi - lo)
        smoothed = (1 - smooth) * out / factor + smooth * out
        medium = ~(wavelen < high_wl) * ~(wavelen > low_wl)
        return torch.where(medium, smoothed, out), 1.0
    if rope_type == 'longrope':
        orig = original_max_position_embeddings or rs.get('original_max_position_embeddings')
        factor = rs.get('factor')
        if not orig:
            orig = max_position_embeddings
        if factor is None:     # Phi-3 style configs give only the two lengths
            factor = max_position_embeddings / orig
        attention_factor = rs.get('attention_factor')
        if attention_factor is None:
            attention_factor = 1.0 if factor <= 1.0 else math.sqrt(1 + math.log(factor) / math.log(orig))
        use_long = seq_len is not None and seq_len > orig
        ext = torch.tensor(rs['long_factor'] if use_long else rs['short_factor'], dtype=torch.float32)
        inv = 1.0 / (ext * base**(torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
        return inv, float(attention_factor)
    raise ValueError(f'unknown rope type {rope_type!r}')


def rotary_dim(config) -> int:
    if config.multi_latent_attention and config.partial_rotary_factor is None:
        head_dim = config.qk_pos_emb_head_dim
    else:
        head_dim = config.kv_channels
    factor = config.partial_rotary_factor if config.partial_rotary_factor is not None else config.rotary_percent
    dim = int(head_dim * factor)
    return dim - (dim % 2)


def get_rope_inv_freq(config, seq_len: Optional[int] = None, base: Optional[float] = None):
    """``(inv_freq, attention_scaling)`` for a :class:`ModelConfig`."""
    rs = config.rope_scaling
    return compute_inv_freq(_rope_type(rs), float(base if base is not None else config.rotary_base), rotary_dim(config),
                            rs, config.max_position_embeddings, seq_len, config.original_max_position_embeddings)


class RotaryEmbedding(torch.nn.Module):
    """Holds ``inv_freq`` (fp32 buffer, not persistent) and builds per-token tables."""

    def __init__(self, config, base: Optional[float] = None, rope_scaling_override='__unset__'):
        super().__init__()
        self.config = config
        self.base = float(base if base is not None else config.rotary_base)
        self.rope_scaling = config.rope_scaling if rope_scaling_override == '__unset__' else rope_scaling_override
        self.rope_type = _rope_type(self.rope_scaling)
        self.dim = rotary_dim(config)
        inv, scale = compute_inv_freq(self.rope_type, self.base, self.dim, self.rope_scaling,
                                      config.max_position_embeddings, None, config.original_max_position_embeddings)
        self.register_buffer('inv_freq', inv, persistent=False)
        self.attention_scaling = float(config.attention_scaling) * float(scale)
        self._cached_seq_len = config.max_position_embeddings or 0
        self._uses_long = False

    def _maybe_update(self, seq_len: int):
        """dynamic NTK grows the base with the sequence; longrope switches factor sets (reference
        ``src/mcore_bridge/model/rope.py:126-168``)."""
        cfg = self.config
        if self.rope_type == 'dynamic':
            if seq_len > self._cached_seq_len or (seq_len <= cfg.max_position_embeddings < self._cached_seq_len):
                inv, _ = compute_inv_freq('dynamic', self.base, self.dim, self.rope_scaling,
                                          cfg.max_position_embeddings, seq_len)
                self.inv_freq.copy_(inv.to(self.inv_freq.device))
                self._cached_seq_len = max(seq_len, cfg.max_position_embeddings)
        elif self.rope_type == 'longrope':
            orig = cfg.original_max_position_embeddings or cfg.max_position_embeddings
            want_long = seq_len > orig
            if want_long != self._uses_long:
                inv, _ = compute_inv_freq('longrope', self.base, self.dim, self.rope_scaling,
                                          cfg.max_position_embeddings, seq_len if want_long else None,
                                          cfg.original_max_position_embeddings)
                self.inv_freq.copy_(inv.to(self.inv_freq.device))
                self._uses_long = want_long

    @torch.no_grad()
    def forward(self, position_ids: torch.Tensor, seq_len: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``position_ids``: ``[T]`` or, for MRoPE, ``[3, T]`` (temporal, height, width)."""
        if seq_len is not None:
            self._maybe_update(seq_len)
        inv = self.inv_freq.float()
        cfg = self.config
        if position_ids.dim() == 2 and cfg.position_embedding_type == 'mrope' and cfg.mrope_section is not None:
            freqs3 = position_ids.float()[:, :, None] * inv[None, None, :]  # [3, T, rot/2]
            sec = list(cfg.mrope_section)
            if cfg.mrope_interleaved:
                freqs = freqs3[0].clone()
                for axis, off in ((1, 1), (2, 2)):
                    idx = slice(off, sec[axis] * 3, 3)
                    freqs[:, idx] = freqs3[axis][:, idx]
            else:
                parts, start = [], 0
                for axis, n in enumerate(sec):
                    parts.append(freqs3[axis % 3][:, start:start + n])
                    start += n
                freqs = torch.cat(parts, dim=-1)
        else:
            if position_ids.dim() == 2:
                position_ids = position_ids[0]
            freqs = position_ids.float()[:, None] * inv[None, :]
        cos, sin = freqs.cos(), freqs.sin()
        if self.attention_scaling != 1.0:
            cos, sin = cos * self.attention_scaling, sin * self.attention_scaling
        return cos.contiguous(), sin.contiguous()
