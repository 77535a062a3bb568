"""Dequantisers for quantised Hugging Face checkpoints: block-scaled fp8, MXFP4, fp4(e2m1)->fp8, packed int4/int8.

Semantics as in reference ``src/mcore_bridge/utils/dequantizer.py:6-152``; formulas written out here.
``GPTBridge.load_weights`` applies them through :func:`add_dequantized_views`, so every family loader sees plain
weight keys whatever the storage format of the checkpoint.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

# e2m1 code -> value (sign bit is bit 3)
_FP4_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


class Fp8Dequantizer:
    """``w = q * scale_inv`` with one scale per ``block_m x block_n`` block (ragged edges allowed)."""

    def __init__(self, block_size: Tuple[Optional[int], Optional[int]] = (None, None)):
        self.block_size = block_size

    def convert(self, quantized: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
        if not isinstance(quantized, torch.Tensor) or not isinstance(scales, torch.Tensor):
            raise TypeError('Fp8Dequantizer expects tensors')
        if quantized.dtype == torch.uint8:
            quantized = quantized.view(torch.float8_e4m3fn)
        q = quantized.to(torch.float32)
        rows, cols = q.shape[-2:]
        srows, scols = scales.shape[-2:]
        bm, bn = self.block_size
        # the usual checkpoints use 128 x 128 blocks; anything else is inferred from the scale grid
        bm = bm or (128 if -(-rows // 128) == srows else -(-rows // srows))
        bn = bn or (128 if -(-cols // 128) == scols else -(-cols // scols))
        s = scales.to(torch.float32)
        s = s.repeat_interleave(bm, dim=-2)[..., :rows, :].repeat_interleave(bn, dim=-1)[..., :, :cols]
        return q * s


def quantize_fp8_blockwise(w: torch.Tensor, block: Tuple[int, int] = (128, 128)):
    """Inverse of :class:`Fp8Dequantizer`: returns ``(fp8 e4m3 tensor, scale_inv)``."""
    bm, bn = block
    rows, cols = w.shape[-2:]
    pr, pc = (-rows) % bm, (-cols) % bn
    wf = torch.nn.functional.pad(w.float(), (0, pc, 0, pr))
    R, C = wf.shape[-2:]
    blocks = wf.reshape(*wf.shape[:-2], R // bm, bm, C // bn, bn)
    amax = blocks.abs().amax(dim=(-3, -1), keepdim=True).clamp(min=1e-12)
    scale_inv = amax / 448.0
    q = (blocks / scale_inv).reshape(*wf.shape[:-2], R, C)[..., :rows, :cols].to(torch.float8_e4m3fn)
    return q, scale_inv.squeeze(-1).squeeze(-2)


class MxFp4Dequantizer:
    """MXFP4: two e2m1 values per byte (low nibble first), one e8m0 scale per 32 values."""

    def convert(self, blocks: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        lut = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=blocks.device)
        b = blocks.to(torch.uint8)
        lo, hi = (b & 0x0F).long(), (b >> 4).long()
        vals = torch.stack((lut[lo], lut[hi]), dim=-1).flatten(-2)         # [..., G, 32]
        exp = scales.to(torch.int32) - 127
        out = torch.ldexp(vals, exp.unsqueeze(-1))
        return out.flatten(-2).to(dtype)


def fp4_e2m1_to_float(packed: torch.Tensor) -> torch.Tensor:
    """``[..., n]`` bytes (int8 / uint8) holding two e2m1 values each, low nibble first -> fp32 ``[..., 2 n]``
    (unscaled; parity: reference ``src/mcore_bridge/utils/dequantizer.py:67-79``)."""
    lut = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=packed.device)
    b = packed.contiguous().view(torch.uint8)
    return torch.stack((lut[(b & 0x0F).long()], lut[(b >> 4).long()]), dim=-1).flatten(-2)


def quantize_mxfp4(w: torch.Tensor):
    """Inverse of :class:`MxFp4Dequantizer` (round to nearest e2m1 value, power-of-two scale per 32 values along the
    last dim): returns ``(blocks uint8 [..., G, 16], scales uint8 [..., G])``.  Used to write MXFP4 checkpoints and
    to build test fixtures."""
    assert w.shape[-1] % 32 == 0
    x = w.float().reshape(*w.shape[:-1], -1, 32)
    amax = x.abs().amax(dim=-1, keepdim=True).clamp(min=2.0 ** -120)
    exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)        # largest magnitude maps inside [-6, 6]
    scaled = x / torch.exp2(exp)
    lut = torch.tensor(_FP4_VALUES[:8], dtype=torch.float32, device=w.device)
    mag = (scaled.abs().unsqueeze(-1) - lut).abs().argmin(dim=-1)     # nearest magnitude code 0..7
    code = (mag + (scaled < 0).long() * 8).to(torch.uint8)
    blocks = (code[..., 0::2] | (code[..., 1::2] << 4)).contiguous()
    return blocks, (exp.squeeze(-1) + 127).to(torch.uint8)


def fp4_to_fp8(packed: torch.Tensor) -> torch.Tensor:
    """Unpacks e2m1 nibbles (low first) into ``float8_e4m3fn`` values; output last dim doubles."""
    lut = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=packed.device)
    b = packed.view(torch.uint8)
    lo, hi = (b & 0x0F).long(), (b >> 4).long()
    return torch.stack((lut[lo], lut[hi]), dim=-1).flatten(-2).to(torch.float8_e4m3fn)


def pack_int_weights(w_int: torch.Tensor, num_bits: int) -> torch.Tensor:
    """Signed integers in ``[-2^(bits-1), 2^(bits-1))`` -> offset-binary values packed into int32 words along the
    last dim (the layout :class:`PackedDequantizer` reads)."""
    per = 32 // num_bits
    cols = w_int.shape[-1]
    pad = (-cols) % per
    u = (w_int.to(torch.int64) + (1 << (num_bits - 1)))
    u = torch.nn.functional.pad(u, (0, pad)).reshape(*w_int.shape[:-1], -1, per)
    shifts = torch.arange(per, dtype=torch.int64, device=w_int.device) * num_bits
    word = (u << shifts).sum(dim=-1)
    word = torch.where(word >= (1 << 31), word - (1 << 32), word)    # two's complement int32
    return word.to(torch.int32)


class PackedDequantizer:
    """compressed-tensors style packed int4 / int8 weights: ``weight_packed`` (int32 words holding
    ``32/bits`` values, offset-binary), ``weight_scale`` per group, optional ``weight_zero_point``."""

    def __init__(self, quantization_config: dict):
        cfg = quantization_config or {}
        groups = cfg.get('config_groups') or {}
        w = {}
        for g in groups.values():
            w = g.get('weights') or {}
            break
        self.num_bits = int(w.get('num_bits', cfg.get('bits', 4)))
        self.group_size = w.get('group_size', cfg.get('group_size', 128))
        self.symmetric = bool(w.get('symmetric', True))

    def unpack(self, packed: torch.Tensor, shape) -> torch.Tensor:
        bits = self.num_bits
        per = 32 // bits
        p = packed.to(torch.int32)
        shifts = torch.arange(per, device=p.device, dtype=torch.int32) * bits
        vals = (p.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
        vals = vals.flatten(-2)[..., :shape[-1]]
        return vals - (1 << (bits - 1))  # offset binary -> signed

    def convert(self, weight_packed: torch.Tensor, weight_scale: torch.Tensor, weight_shape,
                weight_zero_point: Optional[torch.Tensor] = None, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        shape = [int(x) for x in (weight_shape.tolist() if isinstance(weight_shape, torch.Tensor) else weight_shape)]
        q = self.unpack(weight_packed, shape).to(torch.float32)
        rows, cols = shape[-2], shape[-1]
        scale = weight_scale.to(torch.float32)
        gs = self.group_size if self.group_size and self.group_size > 0 else cols
        s = scale.repeat_interleave(gs, dim=-1)[..., :cols] if scale.shape[-1] != cols else scale
        if weight_zero_point is not None and not self.symmetric:
            packed_zp = weight_zero_point.dtype == torch.int32
            zp = self.unpack(weight_zero_point, [rows, scale.shape[-1]]).float() if packed_zp \
                else weight_zero_point.float()
            q = q - zp.repeat_interleave(gs, dim=-1)[..., :cols]
        return (q * s).to(dtype)


def add_dequantized_views(sd: dict, quantization_config: Optional[dict], lazy_cls) -> dict:
    """Adds, next to the stored tensors of a quantised checkpoint, lazily dequantised entries under the plain keys
    the loaders ask for (parity: reference ``src/mcore_bridge/bridge/gpt_bridge.py:874-877,930-937,1157-1187``):

    * MXFP4 (GPT-OSS experts): ``X_blocks`` + ``X_scales`` -> ``X``, transposed to the input-major layout of the
      bf16 checkpoints (``[E, in, out]``);
    * compressed-tensors: ``M.weight_packed`` + ``M.weight_scale`` + ``M.weight_shape`` (+ ``M.weight_zero_point``)
      -> ``M.weight``.

    ``lazy_cls`` is the ``LazyTensor`` class (passed in to keep this module free of I/O imports)."""
    out = dict(sd)
    mx = MxFp4Dequantizer()
    for key in sd:
        if key.endswith('_blocks') and key[:-len('_blocks')] + '_scales' in sd:
            base = key[:-len('_blocks')]
            if base in sd:
                continue

            def load_mx(base=base):
                w = mx.convert(sd[base + '_blocks'].load(), sd[base + '_scales'].load())
                return w.transpose(-1, -2).contiguous() if w.dim() == 3 else w

            out[base] = lazy_cls(loader=load_mx)
    packed = [k for k in sd if k.endswith('.weight_packed')]
    if packed:
        deq = PackedDequantizer(quantization_config or {})
        for key in packed:
            mod = key[:-len('.weight_packed')]
            if mod + '.weight' in sd:
                continue

            def load_packed(mod=mod):
                zp = sd.get(mod + '.weight_zero_point')
                return deq.convert(sd[mod + '.weight_packed'].load(), sd[mod + '.weight_scale'].load(),
                                   sd[mod + '.weight_shape'].load(), None if zp is None else zp.load(),
                                   dtype=torch.float32)

            out[mod + '.weight'] = lazy_cls(loader=load_packed)
    return out
