"""Vocab-parallel cross entropy and the fused linear + cross-entropy head.

* :func:`vocab_parallel_cross_entropy` — logits sharded on the vocab dim; max / sum-exp / target-logit
  reduced over the tensor-parallel group (parity: the ``compute_language_model_loss`` call at reference
  ``src/mcore_bridge/model/gpt_model.py:577``).
* :func:`fused_linear_cross_entropy` — never materialises the logits.  On a GPU the head GEMM's epilogue reduces
  every 128 x 256 accumulator tile to per-row (max, sum-exp) partials and picks out the label's logit
  (``csrc/gemm``, ``EPI_CE_STATS``); the partials of a row are combined, the tensor-parallel ranks exchange their
  ``[T]`` statistics through peer memory (``parallel/dp_comm.py`` all-gather kernel; ``torch.distributed`` elsewhere)
  and the loss follows.  Backward runs the head GEMM again per token chunk with an epilogue that writes the
  gradient of the logits directly in bf16 (``EPI_CE_GRAD``) and feeds it to the two gradient GEMMs.  Only ``[T]``
  statistics are kept between forward and backward.  On CPU the same chunked algorithm runs on torch ops.

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


_STATS_WS = {}


def _reduce_stats_peer(m, s, tgt, group_name):
    """Same combination as :func:`_reduce_stats`, with the ranks' ``[3, T]`` statistics exchanged by the in-tree
    peer-memory all-gather kernel instead of two NCCL all-reduces."""
    from ..parallel import dp_comm
    n, r = ps.get_world_size(group_name), ps.get_rank_in(group_name)
    T = m.numel()
    per = 3 * T
    per_al = (per + 3) // 4 * 4                     # 16-byte multiples per rank
    cur = _STATS_WS.get(group_name)
    if cur is None or cur[1].numel() < n * per_al:
        if cur is not None:
            torch.cuda.synchronize()
        cur = _STATS_WS[group_name] = dp_comm.allocate(group_name, n * max(per_al, 1 << 16), torch.float32)
    ws, flat = cur
    mine = flat[r * per_al:r * per_al + per].view(3, T)
    mine[0].copy_(m)
    mine[1].copy_(s)
    mine[2].copy_(tgt)
    dp_comm.all_gather_(ws, flat, 0, n * per_al)
    allr = flat[:n * per_al].view(n, per_al)[:, :per].view(n, 3, T)
    gm = allr[:, 0].max(dim=0).values
    ssum = (allr[:, 1] * torch.exp(allr[:, 0] - gm)).sum(0)
    return gm + torch.log(ssum), allr[:, 2].sum(0)


def _combine(m, s, tgt, group_name, group):
    if group is not None and m.is_cuda:
        from ..parallel import dp_comm
        if dp_comm.usable(group_name, m.device):
            return _reduce_stats_peer(m, s, tgt, group_name)
    return _reduce_stats(m, s, tgt, group)


def _head_kernel_ok(h2, weight) -> bool:
    return (h2.is_cuda and h2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _lib.available()
            and h2.shape[1] % 8 == 0 and weight.is_contiguous())


def _head_stats(h2, weight, lab, vocab_start):
    """(max, sum exp, label logit) of every row over the local vocabulary shard, from the GEMM epilogue."""
    T, H = h2.shape
    vl = weight.shape[0]
    tiles_n = (vl + 255) // 256
    part = torch.empty((T, tiles_n, 2), dtype=torch.float32, device=h2.device)
    tgt = torch.zeros(T, dtype=torch.float32, device=h2.device)
    rc = _lib.lib().mcb_gemm_ce_bf16(_lib.ptr(h2), _ll(h2.stride(0)), _lib.ptr(weight), _ll(weight.stride(0)), _int(T),
                                     _int(vl), _int(H), _lib.ptr(lab), _int(vocab_start), _lib.ptr(part), _lib.ptr(tgt),
                                     None, None, None, _ll(0), _int(0), _lib.ptr(_lib.status_word(h2.device)),
                                     _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_gemm_ce_bf16')
    m_t, s_t = part[..., 0], part[..., 1]
    m = m_t.max(dim=1).values
    s = (s_t * torch.exp(m_t - m[:, None])).sum(1)
    return m, s, tgt


def _head_dlogits(h2, weight, lab, vocab_start, lse, g):
    T, H = h2.shape
    vl = weight.shape[0]
    d = torch.empty((T, vl), dtype=torch.bfloat16, device=h2.device)
    rc = _lib.lib().mcb_gemm_ce_bf16(_lib.ptr(h2), _ll(h2.stride(0)), _lib.ptr(weight), _ll(weight.stride(0)), _int(T),
                                     _int(vl), _int(H), _lib.ptr(lab), _int(vocab_start), None, None, _lib.ptr(lse),
                                     _lib.ptr(g), _lib.ptr(d), _ll(d.stride(0)), _int(1),
                                     _lib.ptr(_lib.status_word(h2.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_gemm_ce_bf16')
    return d


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
        if h2.stride(1) != 1 or h2.stride(0) % 8:
            h2 = h2.contiguous()
        if _head_kernel_ok(h2, weight):
            m, s, tgt = _head_stats(h2, weight, lab, r * vl)
            lse_all, tgt = _combine(m, s, tgt, group_name, group)
            ctx.save_for_backward(h2, weight, lab, lse_all)
            ctx.meta = (group_name, chunk, r * vl, h.shape, labels.shape)
            return (lse_all - tgt).view(labels.shape)
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
        fused = _head_kernel_ok(h2, weight)
        for s0 in range(0, T, chunk):
            s1 = min(T, s0 + chunk)
            if fused:
                d = _head_dlogits(h2[s0:s1], weight, lab[s0:s1], vstart, lse[s0:s1], g[s0:s1])
            else:
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
