"""Vocab-parallel cross entropy and the fused linear + cross-entropy head.

* :func:`vocab_parallel_cross_entropy` — logits sharded on the vocab dim; max / sum-exp / target-logit
  reduced over the tensor-parallel group (parity: the ``compute_language_model_loss`` call at reference
  ``src/mcore_bridge/model/gpt_model.py:577``).
* :func:`fused_linear_cross_entropy` — never materialises ``[T, V]``: the head GEMM runs per token chunk,
  the softmax statistics come from a one-pass kernel over the chunk, and backward recomputes the chunk's
  logits, turns them into ``dlogits`` in place and feeds the two gradient GEMMs.  Only ``[T]`` statistics are
  kept between forward and backward.

Both return the per-token loss ``[T]`` in fp32 (the caller masks and averages).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..parallel import state as ps
from . import _lib, gemm

_ll, _int, _f = ctypes.c_longlong, ctypes.c_int, ctypes.c_float


def _tp_info(group: str):
    n = ps.get_world_size(group)
    r = ps.get_rank_in(group) if n > 1 else 0
    return n, r, (ps.get_group(group) if n > 1 else None)


def _stats_torch(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int):
    """Per-row (max, sum exp(l - max), target logit or 0) over the local vocab shard."""
    lf = logits.float()
    vl = lf.shape[-1]
    m = lf.max(dim=-1).values
    s = torch.exp(lf - m[:, None]).sum(-1)
    local = labels - vocab_start
    ok = (local >= 0) & (local < vl)
    tgt = lf.gather(1, local.clamp(0, vl - 1)[:, None]).squeeze(1)
    tgt = torch.where(ok, tgt, torch.zeros_like(tgt))
    return m, s, tgt


def _stats(logits, labels, vocab_start):
    if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16) and _lib.available():
        rows, vl = logits.shape
        m = torch.empty(rows, dtype=torch.float32, device=logits.device)
        s = torch.empty_like(m)
        t = torch.empty_like(m)
        rc = _lib.lib().mcb_ce_stats(_lib.ptr(logits), _int(int(logits.dtype == torch.float32)), _ll(logits.stride(0)),
                                     _lib.ptr(labels), _ll(rows), _int(vl), _int(vocab_start), _lib.ptr(m),
                                     _lib.ptr(s), _lib.ptr(t), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_ce_stats')
        return m, s, t
    return _stats_torch(logits, labels, vocab_start)


def _reduce_stats(m, s, tgt, group):
    """Combine per-shard softmax statistics across the tensor-parallel group -> (lse, target logit)."""
    if group is not None:
        gm = m.clone()
        dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=group)
        packed = torch.stack([s * torch.exp(m - gm), tgt])
        dist.all_reduce(packed, group=group)
        s, tgt, m = packed[0], packed[1], gm
    return m + torch.log(s), tgt


def _dlogits(logits, labels, vocab_start, lse, g, out_dtype):
    """``(softmax - onehot) * g`` for the local shard."""
    if logits.is_cuda and _lib.available() and logits.dtype in (torch.float32, torch.bfloat16):
        rows, vl = logits.shape
        out = torch.empty((rows, vl), dtype=torch.bfloat16, device=logits.device) if out_dtype == torch.bfloat16 \
            else torch.empty((rows, vl), dtype=torch.float32, device=logits.device)
        rc = _lib.lib().mcb_ce_dlogits(_lib.ptr(logits), _int(int(logits.dtype == torch.float32)),
                                       _ll(logits.stride(0)), _lib.ptr(labels), _lib.ptr(lse), _lib.ptr(g), _ll(rows),
                                       _int(vl), _int(vocab_start), _lib.ptr(out),
                                       _int(int(out.dtype == torch.float32)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_ce_dlogits')
        return out
    lf = logits.float()
    vl = lf.shape[-1]
    p = torch.exp(lf - lse[:, None])
    local = labels - vocab_start
    ok = (local >= 0) & (local < vl)
    p[torch.arange(p.shape[0], device=p.device)[ok], local[ok]] -= 1.0
    return (p * g[:, None]).to(out_dtype)


class _VocabParallelCE(torch.autograd.Function):

    @staticmethod
    def forward(ctx, logits, labels, group_name):
        n, r, group = _tp_info(group_name)
        vl = logits.shape[-1]
        l2 = logits.reshape(-1, vl)
        lab = labels.reshape(-1).to(torch.int64)
        m, s, tgt = _stats(l2, lab, r * vl)
        lse, tgt = _reduce_stats(m, s, tgt, group)
        ctx.save_for_backward(l2, lab, lse)
        ctx.vocab_start, ctx.shape = r * vl, logits.shape
        return (lse - tgt).view(labels.shape)

    @staticmethod
    def backward(ctx, g):
        l2, lab, lse = ctx.saved_tensors
        d = _dlogits(l2, lab, ctx.vocab_start, lse, g.reshape(-1).float().contiguous(), l2.dtype)
        return d.view(ctx.shape), None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, group: str = 'tp') -> torch.Tensor:
    """``logits [..., V/tp]``, ``labels [...]`` (global ids) -> per-token loss (fp32)."""
    return _VocabParallelCE.apply(logits, labels, group)


class _FusedLinearCE(torch.autograd.Function):

    @staticmethod
    def forward(ctx, h, weight, labels, group_name, chunk):
        n, r, group = _tp_info(group_name)
        vl, H = weight.shape
        h2 = h.reshape(-1, H)
        lab = labels.reshape(-1).to(torch.int64)
        T = h2.shape[0]
        loss = torch.empty(T, dtype=torch.float32, device=h.device)
        lse_all = torch.empty(T, dtype=torch.float32, device=h.device)
        ldt = torch.float32
        for s0 in range(0, T, chunk):
            s1 = min(T, s0 + chunk)
            logits = gemm.mm_nt(h2[s0:s1], weight, out_dtype=ldt)
            m, s, tgt = _stats(logits, lab[s0:s1], r * vl)
            lse, tgt = _reduce_stats(m, s, tgt, group)
            loss[s0:s1] = lse - tgt
            lse_all[s0:s1] = lse
            del logits
        ctx.save_for_backward(h2, weight, lab, lse_all)
        ctx.meta = (group_name, chunk, r * vl, h.shape, labels.shape)
        return loss.view(labels.shape)

    @staticmethod
    def backward(ctx, g):
        h2, weight, lab, lse = ctx.saved_tensors
        group_name, chunk, vstart, hshape, _ = ctx.meta
        n, r, group = _tp_info(group_name)
        T, H = h2.shape
        g = g.reshape(-1).float().contiguous()
        dh = torch.empty_like(h2)
        mg = getattr(weight, 'main_grad', None)
        dw = None
        need_dw = ctx.needs_input_grad[1]
        if need_dw and mg is None:
            dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        ddt = h2.dtype if h2.dtype == torch.bfloat16 else torch.float32
        for s0 in range(0, T, chunk):
            s1 = min(T, s0 + chunk)
            logits = gemm.mm_nt(h2[s0:s1], weight, out_dtype=torch.float32)
            d = _dlogits(logits, lab[s0:s1], vstart, lse[s0:s1], g[s0:s1], ddt)
            del logits
            gemm.mm_nn(d, weight, out=dh[s0:s1])
            if need_dw:
                gemm.mm_tn(d, h2[s0:s1], out=mg if mg is not None else dw, accumulate=True)
            del d
        # dh is this vocab shard's partial gradient: the caller's input mapping (copy-to-region or
        # sequence-parallel gather) sums it over the tensor-parallel group in its own backward.
        if need_dw and mg is not None:
            hook = getattr(weight, 'grad_ready_hook', None)
            if hook is not None:
                hook()
        return dh.view(hshape), (dw.to(weight.dtype) if dw is not None else None), None, None, None


def fused_linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, group: str = 'tp',
                               chunk: int = 4096) -> torch.Tensor:
    """``h [T, H]`` (full sequence on every TP rank), ``weight [V/tp, H]``, ``labels [T]`` -> loss ``[T]`` fp32."""
    return _FusedLinearCE.apply(h, weight, labels, group, chunk)
