"""Rotary embedding application and the fused QKV post-processing op.

* :func:`apply_rope` — rotate the first ``rot`` dims of ``[T, heads, d]`` with per-token tables
  (rotate-half or interleaved pairs; inverse rotation by negating ``sin``).
* :func:`qkv_split_norm_rope` — split a packed QKV projection per query group, per-head RMSNorm on
  q/k, rope, and write separate q/k/v(/gate) tensors in one pass (CUDA: ``csrc/elementwise/qkv_rope.cu``).

The tables are per token, ``[T, rot/2]`` fp32, so packed sequences, context-parallel chunks, MRoPE
sections and attention scaling (``mscale`` folded into cos/sin, reference
``src/mcore_bridge/model/modules/transformer_layer.py:249-278``) are the table builder's business.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from .norm import rmsnorm_ref

_ll, _int, _f = ctypes.c_longlong, ctypes.c_int, ctypes.c_float


def apply_rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """``x``: ``[T, heads, d]``; ``cos``/``sin``: ``[T, rot/2]``.  Dims past ``rot`` pass through."""
    rot = cos.shape[-1] * 2
    xr, xp = x[..., :rot].float(), x[..., rot:]
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    if interleaved:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).flatten(-2)
    else:
        x1, x2 = xr[..., :rot // 2], xr[..., rot // 2:]
        o = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)
    return torch.cat((o.to(x.dtype), xp), dim=-1)


def apply_rope(x, cos, sin, interleaved: bool = False, inverse: bool = False):
    if inverse:
        sin = -sin
    return apply_rope_ref(x, cos, sin, interleaved)


def qkv_split_norm_rope_ref(qkv, wq, wk, cos, sin, ng, qpg, d, has_gate, interleaved, eps, zero_centered):
    T = qkv.shape[0]
    per_group = qpg * (2 if has_gate else 1) + 2
    x = qkv.reshape(T, ng, per_group, d)
    nqs = qpg * (2 if has_gate else 1)
    qs = x[:, :, :nqs]
    k = x[:, :, nqs]
    v = x[:, :, nqs + 1]
    gate = None
    if has_gate:
        gate = qs[:, :, 1::2].reshape(T, ng * qpg, d)
        q = qs[:, :, 0::2].reshape(T, ng * qpg, d)
    else:
        q = qs.reshape(T, ng * qpg, d)
    if wq is not None:
        q = rmsnorm_ref(q, wq, eps, zero_centered)
        k = rmsnorm_ref(k, wk, eps, zero_centered)
    if cos is not None:
        q = apply_rope_ref(q, cos, sin, interleaved)
        k = apply_rope_ref(k, cos, sin, interleaved)
    return q.contiguous(), k.contiguous(), v.contiguous(), (gate.contiguous() if gate is not None else None)


class _QkvCuda(torch.autograd.Function):

    @staticmethod
    def forward(ctx, qkv, wq, wk, cos, sin, ng, qpg, d, has_gate, interleaved, eps, zero_centered):
        T = qkv.shape[0]
        if qkv.stride(-1) != 1:
            qkv = qkv.contiguous()
        nq = ng * qpg
        dev, dt = qkv.device, qkv.dtype
        q = torch.empty((T, nq, d), dtype=dt, device=dev)
        k = torch.empty((T, ng, d), dtype=dt, device=dev)
        v = torch.empty((T, ng, d), dtype=dt, device=dev)
        gate = torch.empty((T, nq, d), dtype=dt, device=dev) if has_gate else None
        rot = 0 if cos is None else cos.shape[-1] * 2
        norm = wq is not None
        rc = _lib.lib().mcb_qkv_split_norm_rope_fwd(
            _lib.ptr(qkv), _lib.ptr(wq), _lib.ptr(wk), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(q), _lib.ptr(k),
            _lib.ptr(v), _lib.ptr(gate), _ll(T), _int(ng), _int(qpg), _int(d), _int(int(has_gate)), _int(rot),
            _int(int(interleaved)), _int(int(norm)), _int(int(zero_centered)), _f(eps), _ll(qkv.stride(0)),
            _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_qkv_split_norm_rope_fwd')
        ctx.save_for_backward(qkv, wq, wk, cos, sin)
        ctx.meta = (ng, qpg, d, has_gate, rot, interleaved, norm, zero_centered, eps)
        if has_gate:
            return q, k, v, gate
        ctx.mark_non_differentiable()
        return q, k, v, None

    @staticmethod
    def backward(ctx, dq, dk, dv, dgate):
        qkv, wq, wk, cos, sin = ctx.saved_tensors
        ng, qpg, d, has_gate, rot, interleaved, norm, zc, eps = ctx.meta
        T = qkv.shape[0]
        dev = qkv.device
        nq = ng * qpg

        def _c(t, shape):
            if t is None:
                return torch.zeros(shape, dtype=qkv.dtype, device=dev)
            return t.contiguous()

        dq, dk, dv = _c(dq, (T, nq, d)), _c(dk, (T, ng, d)), _c(dv, (T, ng, d))
        if has_gate:
            dgate = _c(dgate, (T, nq, d))
        dqkv = torch.empty_like(qkv)
        dwq = torch.zeros(d, dtype=torch.float32, device=dev) if norm else None
        dwk = torch.zeros(d, dtype=torch.float32, device=dev) if norm else None
        # per-CTA partial sums of the norm-weight gradients, added in a fixed order (bit-reproducible)
        part = torch.empty((_lib.lib().mcb_qkv_bwd_partial_rows(_ll(T)), 2, d), dtype=torch.float32,
                           device=dev) if norm else None
        rc = _lib.lib().mcb_qkv_split_norm_rope_bwd(
            _lib.ptr(qkv), _lib.ptr(wq), _lib.ptr(wk), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(dq), _lib.ptr(dk),
            _lib.ptr(dv), _lib.ptr(dgate if has_gate else None), _lib.ptr(dqkv), _lib.ptr(dwq), _lib.ptr(dwk),
            _lib.ptr(part), _ll(T),
            _int(ng), _int(qpg), _int(d), _int(int(has_gate)), _int(rot), _int(int(interleaved)), _int(int(norm)),
            _int(int(zc)), _f(eps), _ll(qkv.stride(0)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_qkv_split_norm_rope_bwd')
        return (dqkv, dwq.to(wq.dtype) if norm else None, dwk.to(wk.dtype) if norm else None, None, None, None, None,
                None, None, None, None, None)


def qkv_split_norm_rope(qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], num_groups: int,
                        q_per_group: int, head_dim: int, has_gate: bool = False, interleaved: bool = False,
                        eps: float = 1e-6, zero_centered: bool = False
                        ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Packed ``[T, ng*(qpg(+gates)+2)*d]`` -> ``q [T,nq,d]``, ``k [T,ng,d]``, ``v [T,ng,d]``, ``gate``."""
    if (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim <= 256 and head_dim % 8 == 0 and _lib.available()
            and (wq is None or wq.dtype == torch.bfloat16)):
        if cos is not None:
            cos, sin = cos.float().contiguous(), sin.float().contiguous()
        return _QkvCuda.apply(qkv, wq, wk, cos, sin, num_groups, q_per_group, head_dim, has_gate, interleaved, eps,
                              zero_centered)
    return qkv_split_norm_rope_ref(qkv, wq, wk, cos, sin, num_groups, q_per_group, head_dim, has_gate, interleaved,
                                   eps, zero_centered)
