"""Binding of the in-tree sm_100a attention kernels (``csrc/attention``).

Forward: ``attn_fwd_sm100.cu`` (tcgen05 / TMEM, two-pass softmax, two softmax warp groups).  Backward:
``attn_bwd_sm100.cu`` (delta, dQ and dK/dV kernels; the dK/dV kernel can split the query heads of a GQA group over
several CTAs when the grid would not fill the GPU).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from . import _lib

_ll, _int, _f = ctypes.c_longlong, ctypes.c_int, ctypes.c_float


def unsupported_reason(q, k, v, causal, window, sinks, softcap) -> Optional[str]:
    """``None`` when the in-tree kernel covers the call, else what it lacks (used for the one-time warning)."""
    if not causal:
        return 'non-causal attention'
    if window is not None and (window[0] is None or int(window[0]) < 0):
        window = None
    if softcap:
        return 'soft-capped scores'
    if q.dtype != torch.bfloat16:
        return f'dtype {q.dtype}'
    if q.shape[-1] not in (64, 128):
        return f'head size {q.shape[-1]}'
    if v.shape[-1] != q.shape[-1]:
        return f'value head size {v.shape[-1]} != query head size {q.shape[-1]}'
    if q.shape[1] % k.shape[1] != 0 or q.shape[0] != k.shape[0]:
        return 'query / key token counts or head counts that do not match'
    return None


def supported(q, k, v, causal, window, sinks, softcap) -> bool:
    return unsupported_reason(q, k, v, causal, window, sinks, softcap) is None and _lib.available()


def seq_start_from_cu(cu_seqlens: Optional[torch.Tensor], T: int, device) -> torch.Tensor:
    """``[T]`` int32: index of the first token of the packed sequence each token belongs to."""
    if cu_seqlens is None:
        return torch.zeros(T, dtype=torch.int32, device=device)
    cu = cu_seqlens.to(device=device, dtype=torch.int64)
    seg = torch.searchsorted(cu[1:].contiguous(), torch.arange(T, device=device), right=True)
    return cu[:-1][seg.clamp(max=cu.numel() - 2)].to(torch.int32)


def _dkv_splits(T: int, nq: int, nkv: int, device) -> int:
    """How many CTAs share one (key tile, kv head) pair in the dK/dV kernel: enough to put at least about three
    CTAs on every SM, limited to divisors of the GQA ratio.  ``MCB200_ATTN_DKV_SPLITS`` overrides it."""
    env = os.environ.get('MCB200_ATTN_DKV_SPLITS')
    qpg = nq // nkv
    if env:
        s = int(env)
        return s if s >= 1 and qpg % s == 0 else 1
    ctas = ((T + 127) // 128) * nkv
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    s = 1
    while ctas * s < 3 * sms and s * 2 <= qpg and qpg % (s * 2) == 0:
        s *= 2
    return s


class _AttnFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, seq_start, cu_seqlens, max_seqlen, scale):
        T, nq, d = q.shape
        nkv = k.shape[1]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty((nq, T), dtype=torch.float32, device=q.device)
        rc = _lib.lib().mcb_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(seq_start), _lib.ptr(o),
                                     _lib.ptr(lse), _int(T), _int(nq), _int(nkv), _int(d), _f(scale),
                                     _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_attn_fwd')
        ctx.save_for_backward(q, k, v, o, lse, seq_start, cu_seqlens)
        ctx.scale, ctx.max_seqlen = scale, max_seqlen
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, seq_start, cu = ctx.saved_tensors
        do = do.contiguous()
        T, nq, d = q.shape
        lib = _lib.lib()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty((nq, T), dtype=torch.float32, device=q.device)
        nkv = k.shape[1]
        splits = _dkv_splits(T, nq, nkv, q.device)
        partial = None
        if splits > 1:
            partial = torch.empty((2, splits, T, nkv, d), dtype=torch.float32, device=q.device)
        rc = lib.mcb_attn_bwd_split(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do),
                                    _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(seq_start), _lib.ptr(dq),
                                    _lib.ptr(dk), _lib.ptr(dv), _int(T), _int(nq), _int(nkv), _int(d),
                                    _f(ctx.scale), _lib.ptr(partial) if partial is not None else None,
                                    _int(splits), _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_attn_bwd_split')
        return dq, dk, dv, None, None, None, None


def attention(q, k, v, cu_seqlens, max_seqlen, scale, seq_start: Optional[torch.Tensor] = None, window=None,
              sinks: Optional[torch.Tensor] = None):
    """Packed causal self-attention.  ``window = (left, _)`` limits every query to its ``left`` most recent
    predecessors (plus itself); ``sinks [nq]`` adds a learnable per-head logit to every row's softmax."""
    T, nq, d = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if seq_start is None:
        seq_start = seq_start_from_cu(cu_seqlens, T, q.device)
    if max_seqlen is None and cu_seqlens is not None:
        max_seqlen = T
    left = None if window is None or window[0] is None or int(window[0]) < 0 else int(window[0])
    if left is None and sinks is None:
        return _AttnFn.apply(q, k, v, seq_start, cu_seqlens, max_seqlen, float(scale))
    k_lo = seq_start
    if left is not None:
        # still non-decreasing, so the kernels' causal fast paths (k_hi = the query itself) apply unchanged
        k_lo = torch.maximum(seq_start, (torch.arange(T, device=q.device, dtype=torch.int32) - left))
    o, _ = attention_ranges(q, k, v, k_lo.contiguous(), None, None, None, scale, sinks)
    return o


# ---------------------------------------------------------------------------------------------------------------
# general masks: per-query inclusive key ranges (context-parallel attention, non-causal packed attention)
# ---------------------------------------------------------------------------------------------------------------
def ranges_supported(q, k, v) -> bool:
    d = q.shape[-1]
    return (q.is_cuda and q.dtype == torch.bfloat16 and d in (64, 128) and v.shape[-1] == d and k.shape[-1] == d
            and q.shape[1] % k.shape[1] == 0 and _lib.available())


class _AttnRangesFn(torch.autograd.Function):
    """``o[i] = softmax over keys k_lo[i]..k_hi[i] of q[i] k^T * scale`` applied to ``v``; queries ``[T, nq, d]`` and
    keys / values ``[Tk, nkv, d]`` may be different token sets.  ``q_lo`` / ``q_hi`` ``[Tk]`` bound, per key, the
    queries that can see it (they only limit the loops of the dK/dV kernel)."""

    @staticmethod
    def forward(ctx, q, k, v, k_lo, k_hi, q_lo, q_hi, scale, sinks=None):
        T, nq, d = q.shape
        Tk, nkv = k.shape[0], k.shape[1]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty((nq, T), dtype=torch.float32, device=q.device)
        sk = None if sinks is None else sinks.detach().float().contiguous()
        rc = _lib.lib().mcb_attn_fwd_ranges(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(k_lo), _lib.ptr(k_hi),
                                            _lib.ptr(sk), _lib.ptr(o), _lib.ptr(lse), _int(T), _int(Tk), _int(nq),
                                            _int(nkv), _int(d), _f(scale), _lib.ptr(_lib.status_word(q.device)),
                                            _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_attn_fwd_ranges')
        ctx.save_for_backward(q, k, v, o, lse, k_lo, k_hi, q_lo, q_hi, sk)
        ctx.scale = scale
        ctx.sink_dtype = None if sinks is None else sinks.dtype
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse, k_lo, k_hi, q_lo, q_hi, sk = ctx.saved_tensors
        do = do.contiguous()
        T, nq, d = q.shape
        Tk, nkv = k.shape[0], k.shape[1]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty((nq, T), dtype=torch.float32, device=q.device)
        splits = _dkv_splits(Tk, nq, nkv, q.device)
        partial = torch.empty((2, splits, Tk, nkv, d), dtype=torch.float32, device=q.device) if splits > 1 else None
        rc = _lib.lib().mcb_attn_bwd_ranges(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(delta), _int(0),
            _lib.ptr(k_lo), _lib.ptr(k_hi), _lib.ptr(q_lo), _lib.ptr(q_hi), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
            _int(T), _int(Tk), _int(nq), _int(nkv), _int(d), _f(ctx.scale), _lib.ptr(partial), _int(splits),
            _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_attn_bwd_ranges')
        dsinks = None
        if sk is not None:
            # the sink is one more softmax column with a zero value vector: d sink_h = -sum_i p_sink(i, h) * delta(i, h)
            dsinks = -(torch.exp(sk[:, None] - lse) * delta).sum(1).to(ctx.sink_dtype)
        return dq, dk, dv, None, None, None, None, None, dsinks


def fwd_ranges_raw(q, k, v, k_lo, k_hi, scale: float):
    """One forward launch without autograd: ``(o [T, nq, d], lse [nq, T])`` of the queries over their key ranges in
    ``k`` / ``v`` (rows with an empty range: ``o = 0``, ``lse = -inf``).  Building block of ring attention."""
    T, nq, d = q.shape
    o = torch.empty_like(q)
    lse = torch.empty((nq, T), dtype=torch.float32, device=q.device)
    rc = _lib.lib().mcb_attn_fwd_ranges(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(k_lo), _lib.ptr(k_hi), None,
                                        _lib.ptr(o), _lib.ptr(lse), _int(T), _int(k.shape[0]), _int(nq),
                                        _int(k.shape[1]), _int(d), _f(scale), _lib.ptr(_lib.status_word(q.device)),
                                        _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_attn_fwd_ranges')
    return o, lse


def bwd_ranges_raw(q, k, v, o, do, lse, delta, k_lo, k_hi, q_lo, q_hi, scale: float):
    """One backward launch without autograd, with the log-sum-exp and ``delta = rowsum(o * do)`` of the *whole*
    attention given (``[nq, T]`` fp32): ``(dq, dk, dv)`` of this block of keys."""
    T, nq, d = q.shape
    Tk, nkv = k.shape[0], k.shape[1]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    splits = _dkv_splits(Tk, nq, nkv, q.device)
    partial = torch.empty((2, splits, Tk, nkv, d), dtype=torch.float32, device=q.device) if splits > 1 else None
    rc = _lib.lib().mcb_attn_bwd_ranges(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(delta), _int(1),
        _lib.ptr(k_lo), _lib.ptr(k_hi), _lib.ptr(q_lo), _lib.ptr(q_hi), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
        _int(T), _int(Tk), _int(nq), _int(nkv), _int(d), _f(scale), _lib.ptr(partial), _int(splits),
        _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_attn_bwd_ranges')
    return dq, dk, dv


def attention_ranges(q, k, v, k_lo, k_hi, q_lo, q_hi, scale: Optional[float] = None,
                     sinks: Optional[torch.Tensor] = None):
    """Returns ``(o [T, nq, d], lse [nq, T])``; all four range tensors are int32 on the device (``k_hi`` / ``q_lo`` /
    ``q_hi`` may all be ``None`` for masks of the causal family: ``k_hi[i] = i`` and a non-decreasing ``k_lo``)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return _AttnRangesFn.apply(q, k, v, k_lo, k_hi, q_lo, q_hi, float(scale), sinks)
