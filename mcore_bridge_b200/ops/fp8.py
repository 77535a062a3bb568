"""Block-scaled fp8 (e4m3) matmuls: 1 x 128 activation blocks, 128 x 128 weight blocks, fp32 scales.

CUDA path: ``csrc/gemm/gemm_fp8_sm100.cu`` (tcgen05 ``kind::f8f6f4`` partial products promoted with their scales in
fp32 registers) plus the two quantisation kernels.  The torch functions below restate the same arithmetic and are the
oracle of the kernels and the CPU path.  The scale convention is the one of ``weight_scale_inv`` checkpoints
(reference ``src/mcore_bridge/bridge/gpt_bridge.py:238-252``, ``src/mcore_bridge/utils/dequantizer.py:6-50``):
``value = fp8 * scale`` with ``scale = amax / 448``.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib, gemm

_int = ctypes.c_int
E4M3_MAX = 448.0
BLOCK = 128


# ------------------------------------------------------------------------------------------------ torch reference
def quantize_1x128_ref(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [M, K]`` -> (``x8 [M, K]`` float8_e4m3fn, ``scales [K/128, M]`` fp32)."""
    M, K = x.shape
    xb = x.float().view(M, K // BLOCK, BLOCK)
    amax = xb.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    x8 = (xb / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(M, K)
    return x8, scale.t().contiguous()


def quantize_128x128_ref(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [N, K]`` -> (``w8 [N, K]``, ``scales [ceil(N/128), K/128]``)."""
    N, K = w.shape
    nb = (N + BLOCK - 1) // BLOCK
    wp = torch.zeros(nb * BLOCK, K, dtype=torch.float32, device=w.device)
    wp[:N] = w.float()
    blocks = wp.view(nb, BLOCK, K // BLOCK, BLOCK)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    w8 = (blocks / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return w8.view(nb * BLOCK, K)[:N].contiguous(), scale.contiguous()


def gemm_blockscaled_ref(a8, sa, b8, sb, out_dtype=torch.bfloat16) -> torch.Tensor:
    """fp32 evaluation of the block-scaled product (dequantise, then matmul)."""
    M, K = a8.shape
    N = b8.shape[0]
    a = a8.float().view(M, K // BLOCK, BLOCK) * sa.t()[..., None]
    sbe = sb.repeat_interleave(BLOCK, dim=0)[:N]                              # [N, K/128]
    b = b8.float().view(N, K // BLOCK, BLOCK) * sbe[..., None]
    return (a.view(M, K) @ b.view(N, K).t()).to(out_dtype)


# ------------------------------------------------------------------------------------------------ CUDA bindings
def _use_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and _lib.available()


def quantize_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    if not _use_cuda(x):
        return quantize_1x128_ref(x)
    M, K = x.shape
    x = x.contiguous()
    x8 = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((K // BLOCK, M), dtype=torch.float32, device=x.device)
    rc = _lib.lib().mcb_quant_fp8_1x128(_lib.ptr(x), _lib.ptr(x8), _lib.ptr(s), _int(M), _int(K), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_quant_fp8_1x128')
    return x8, s


def quantize_128x128(w: torch.Tensor, with_transpose: bool = False):
    """Returns ``(w8, scales)`` or, with ``with_transpose``, ``(w8, scales, w8t [K, N], scales_t [K/128, N/128])``."""
    N, K = w.shape
    if not _use_cuda(w):
        w8, s = quantize_128x128_ref(w)
        if not with_transpose:
            return w8, s
        return w8, s, w8.t().contiguous(), s.t().contiguous()
    w = w.contiguous()
    nb = (N + BLOCK - 1) // BLOCK
    w8 = torch.empty((N, K), dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((nb, K // BLOCK), dtype=torch.float32, device=w.device)
    w8t = st = None
    if with_transpose:
        assert N % 16 == 0, 'the transposed copy needs N to be a multiple of 16'
        w8t = torch.empty((K, N), dtype=torch.float8_e4m3fn, device=w.device)
        st = torch.empty((K // BLOCK, nb), dtype=torch.float32, device=w.device)
    rc = _lib.lib().mcb_quant_fp8_128x128(_lib.ptr(w), _lib.ptr(w8), _lib.ptr(s),
                                          _lib.ptr(w8t) if w8t is not None else None,
                                          _lib.ptr(st) if st is not None else None, _int(N), _int(K), _int(N),
                                          _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_quant_fp8_128x128')
    return (w8, s, w8t, st) if with_transpose else (w8, s)


def gemm_blockscaled(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """``C [M, N] = dequant(a8) @ dequant(b8)^T`` in bf16."""
    if not _use_cuda(a8):
        return gemm_blockscaled_ref(a8, sa, b8, sb)
    M, K = a8.shape
    N = b8.shape[0]
    c = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
    rc = _lib.lib().mcb_gemm_fp8_blockscaled(_lib.ptr(a8), _lib.ptr(sa), _lib.ptr(b8), _lib.ptr(sb), _lib.ptr(c),
                                             _int(M), _int(N), _int(K), _lib.ptr(_lib.status_word(a8.device)),
                                             _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_gemm_fp8_blockscaled')
    return c


# ------------------------------------------------------------------------------------------------ weights cache
def eligible(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    N, K = weight.shape
    return x2.dtype == torch.bfloat16 and K % BLOCK == 0 and N % BLOCK == 0


def quantized_weight(weight: torch.Tensor):
    """fp8 copies of a bf16 weight (and of its transpose for the data gradient), re-made only when the weight
    changed: the cache key is the tensor's version counter, which every in-place optimizer update bumps."""
    cache = getattr(weight, '_fp8_cache', None)
    ver = weight._version
    if cache is not None and cache[0] == ver:
        return cache[1]
    q = quantize_128x128(weight.detach(), with_transpose=True)
    try:
        weight._fp8_cache = (ver, q)
    except Exception:
        pass
    return q


def mm_nt(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x2 [M, K] @ weight[N, K]^T`` with both operands quantised on the fly."""
    w8, sw, _, _ = quantized_weight(weight)
    x8, sx = quantize_1x128(x2)
    y = gemm_blockscaled(x8, sx, w8, sw)
    return y if bias is None else y + bias


def mm_nn(dy2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``dy2 [M, N] @ weight[N, K]`` (data gradient) through the transposed fp8 copy of the weight."""
    _, _, w8t, swt = quantized_weight(weight)
    d8, sd = quantize_1x128(dy2)
    return gemm_blockscaled(d8, sd, w8t, swt)
