"""Gated activations: SwiGLU, quick-GEGLU (clamped, offset — gpt-oss), GEGLU-tanh; forward + backward.

Input is ``[rows, 2F]`` laid out ``[gate | up]`` (the fc1 layout the bridge writes); output ``[rows, F]``.
An optional per-row probability multiplies the output (MoE experts weight their output by the router
probability before the second GEMM, so the combine is a plain sum).
CUDA: ``csrc/elementwise/norm_act.cu``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

_ll, _int, _f = ctypes.c_longlong, ctypes.c_int, ctypes.c_float
KINDS = {'swiglu': 0, 'quick_geglu': 1, 'geglu_tanh': 2}


def glu_ref(x, kind='swiglu', probs=None, clamp: float = 0.0, offset: float = 0.0):
    g, u = x.float().chunk(2, dim=-1)
    if clamp and clamp > 0:
        g = g.clamp(max=clamp)
        u = u.clamp(min=-clamp, max=clamp)
    if kind == 'swiglu':
        a = F.silu(g)
    elif kind == 'quick_geglu':
        a = g * torch.sigmoid(1.702 * g)
    else:
        a = F.gelu(g, approximate='tanh')
    y = a * (u + offset)
    if probs is not None:
        y = y * probs.float().unsqueeze(-1)
    return y.to(x.dtype)


class _GluCuda(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, probs, kind, clamp, offset):
        F2 = x.shape[-1]
        Fh = F2 // 2
        x2 = x.reshape(-1, F2)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        rows = x2.shape[0]
        out = torch.empty((rows, Fh), dtype=x.dtype, device=x.device)
        pr = None if probs is None else probs.reshape(-1).float().contiguous()
        rc = _lib.lib().mcb_glu_fwd(_lib.ptr(x2), _lib.ptr(pr), _lib.ptr(out), _ll(rows), _int(Fh), _ll(x2.stride(0)),
                                    _int(kind), _f(clamp), _f(offset), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_glu_fwd')
        ctx.save_for_backward(x2, pr)
        ctx.args = (kind, clamp, offset, x.shape, None if probs is None else (probs.shape, probs.dtype))
        return out.view(*x.shape[:-1], Fh)

    @staticmethod
    def backward(ctx, dout):
        x2, pr = ctx.saved_tensors
        kind, clamp, offset, shape, pmeta = ctx.args
        rows, F2 = x2.shape
        Fh = F2 // 2
        d2 = dout.reshape(rows, Fh).contiguous()
        din = torch.empty((rows, F2), dtype=x2.dtype, device=x2.device)
        dpr = torch.empty(rows, dtype=torch.float32, device=x2.device) if pr is not None else None
        rc = _lib.lib().mcb_glu_bwd(_lib.ptr(x2), _lib.ptr(pr), _lib.ptr(d2), _lib.ptr(din), _lib.ptr(dpr), _ll(rows),
                                    _int(Fh), _ll(x2.stride(0)), _int(kind), _f(clamp), _f(offset), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_glu_bwd')
        dprobs = None
        if pmeta is not None:
            dprobs = dpr.view(pmeta[0]).to(pmeta[1])
        return din.view(shape), dprobs, None, None, None


def glu(x: torch.Tensor, kind: str = 'swiglu', probs: Optional[torch.Tensor] = None, clamp: float = 0.0,
        offset: float = 0.0) -> torch.Tensor:
    clamp = float(clamp or 0.0)
    if x.is_cuda and x.dtype == torch.bfloat16 and (x.shape[-1] // 2) % 8 == 0 and _lib.available():
        return _GluCuda.apply(x, probs, KINDS[kind], clamp, float(offset))
    return glu_ref(x, kind, probs, clamp, offset)


def swiglu(x: torch.Tensor, probs: Optional[torch.Tensor] = None) -> torch.Tensor:
    return glu(x, 'swiglu', probs)
