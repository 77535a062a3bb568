"""RMSNorm (plain / zero-centred gamma / per-head), forward + backward.

CUDA: ``csrc/elementwise/norm_act.cu``.  The torch path is the CPU oracle; its math follows the
zero-centred definition the reference spells out in ``src/mcore_bridge/model/gpts/qwen3_next.py:87-95``
(``x * rsqrt(mean(x^2) + eps) * (1 + w)`` computed in fp32).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_ll, _int, _f = ctypes.c_longlong, ctypes.c_int, ctypes.c_float


def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float, zero_centered: bool = False) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + 1.0 if zero_centered else w.float()
    return (y * wf).to(x.dtype)


class _RMSNormCuda(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, w, eps, zero_centered):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty((rows, H), dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _lib.lib().mcb_rmsnorm_fwd(_lib.ptr(x2), None, _lib.ptr(w), _lib.ptr(y), None, _lib.ptr(rstd),
                                        _ll(rows), _int(H), _ll(x2.stride(0)), _f(eps), _int(int(zero_centered)),
                                        _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_rmsnorm_fwd')
        ctx.save_for_backward(x2, w, rstd)
        ctx.eps, ctx.zc, ctx.shape = eps, zero_centered, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        H = x2.shape[-1]
        rows = x2.shape[0]
        dy2 = dy.reshape(rows, H).contiguous()
        dx = torch.empty((rows, H), dtype=x2.dtype, device=x2.device)
        dw = part = None
        if ctx.needs_input_grad[1]:
            # per-CTA partial rows summed in a fixed order: the weight gradient repeats bit for bit
            dw = torch.zeros(H, dtype=torch.float32, device=x2.device)
            part = torch.empty((_lib.lib().mcb_rmsnorm_bwd_partial_rows(_ll(rows), _int(H)), H), dtype=torch.float32,
                               device=x2.device)
        rc = _lib.lib().mcb_rmsnorm_bwd_det(_lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(w), _lib.ptr(rstd), None,
                                            _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(part), _ll(rows), _int(H),
                                            _ll(x2.stride(0)), _f(ctx.eps), _int(int(ctx.zc)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_rmsnorm_bwd_det')
        return dx.view(ctx.shape), (dw.to(w.dtype) if dw is not None else None), None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, zero_centered: bool = False) -> torch.Tensor:
    """Normalises the last dimension.  ``x`` may be ``[..., H]`` (per-head norm: pass ``[..., heads, d]``)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
            and x.shape[-1] <= 16384 and _lib.available():
        return _RMSNormCuda.apply(x, w, eps, zero_centered)
    return rmsnorm_ref(x, w, eps, zero_centered)


def layernorm_ref(x, w, b, eps):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(),
                                          eps).to(x.dtype)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x / sqrt(sum(x^2) + eps)`` over the last dim (q/k normalisation of gated DeltaNet)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)
