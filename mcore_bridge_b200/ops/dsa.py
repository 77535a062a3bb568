"""DSA (DeepSeek sparse attention): lightning-indexer scores, top-k sparse attention, indexer KL loss.

Torch implementations (the oracle, and the path used where the CUDA kernels do not apply):

* :func:`index_scores` — ``score[s, t] = sum_h w[s, h] * relu(q[s, h] . k[t])`` in fp32, ``-inf`` outside ``mask``.
* :func:`sparse_attention` — softmax attention restricted to each query's selected keys (and the causal /
  same-sequence mask).  Parity: Transformers ``GlmMoeDsaAttention`` builds the same additive mask
  (``modeling_glm_moe_dsa.py``, "Build combined DSA + causal mask").
* :func:`indexer_kl_loss` — KL(attention distribution summed over heads || softmax(index scores)), optionally
  restricted to the selected keys (``dsa_indexer_use_sparse_loss``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def index_scores(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, mask: torch.Tensor,
                 chunk: int = 2048) -> torch.Tensor:
    """``q [T, h, d]``, ``k [Tk, d]``, ``w [T, h]`` (scales folded in), ``mask [T, Tk]`` bool -> ``[T, Tk]`` fp32."""
    T = q.shape[0]
    out = torch.empty(T, k.shape[0], dtype=torch.float32, device=q.device)
    kf = k.float()
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        sc = torch.einsum('shd,td->sht', q[s:e].float(), kf)
        out[s:e] = torch.einsum('sht,sh->st', torch.relu(sc), w[s:e].float())
    return out.masked_fill(~mask, float('-inf'))


def topk_mask(idx: torch.Tensor, Tk: int) -> torch.Tensor:
    m = torch.zeros(idx.shape[0], Tk, dtype=torch.bool, device=idx.device)
    m.scatter_(1, idx, True)
    return m


def sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, idx: torch.Tensor, mask: torch.Tensor,
                     scale: float, need_probs: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``q [T, h, dq]``, ``k [Tk, h, dq]``, ``v [Tk, h, dv]``, ``idx [T, topk]`` -> ``o [T, h, dv]``.

    A selected index that violates ``mask`` (possible when a row has fewer than top-k visible keys) is ignored.
    """
    T, Tk = q.shape[0], k.shape[0]
    keep = topk_mask(idx, Tk) & mask
    s = torch.einsum('shd,thd->hst', q.float(), k.float()) * scale
    s = s.masked_fill(~keep[None], float('-inf'))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum('hst,thd->shd', p, v.float()).to(q.dtype)
    return o, (p if need_probs else None)


def indexer_kl_loss(scores: torch.Tensor, attn_probs: torch.Tensor, mask: torch.Tensor,
                    idx: Optional[torch.Tensor] = None, head_group: Optional[str] = None,
                    token_share: int = 1) -> torch.Tensor:
    """``scores [T, Tk]`` (with ``-inf`` outside the mask), ``attn_probs [h, T, Tk]`` -> scalar KL.

    ``head_group``: the heads are split over this process group (tensor parallelism): the target distribution is the
    sum over all of them.  ``token_share``: the queries are 1 / ``token_share`` of the token stream (context
    parallelism): the result is this rank's share of the mean over the whole stream, like the other auxiliary losses."""
    target = attn_probs.sum(0)
    if head_group is not None:
        import torch.distributed as dist

        from ..parallel import state as ps
        if ps.get_world_size(head_group) > 1:
            target = target.clone()
            dist.all_reduce(target, group=ps.get_group(head_group))
    keep = mask if idx is None else (topk_mask(idx, scores.shape[1]) & mask)
    target = target.masked_fill(~keep, 0.0)
    target = target / target.sum(-1, keepdim=True).clamp(min=1e-20)
    logp = torch.log_softmax(scores.masked_fill(~keep, float('-inf')), dim=-1)
    logp = torch.where(keep, logp, torch.zeros_like(logp))
    kl = (target * (torch.log(target.clamp(min=1e-20)) - logp)).sum(-1)
    return kl.mean() / token_share


# ------------------------------------------------------------------------------------------------ CUDA kernels
def cuda_indexer_supported(q: torch.Tensor, k: torch.Tensor) -> bool:
    from . import _lib
    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 128
            and q.shape[0] == k.shape[0] and q.shape[0] % 4 == 0 and _lib.available())


def index_scores_cuda(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, seq_start: torch.Tensor) -> torch.Tensor:
    """Lightning-indexer scores on the tcgen05 kernel (``csrc/dsa/dsa_indexer_sm100.cu``): ``[T, T]`` fp32 with
    ``-inf`` outside the causal, same-sequence region described by ``seq_start``.  No gradient."""
    import ctypes

    from . import _lib
    T, H, D = q.shape
    out = torch.full((T, T), float('-inf'), dtype=torch.float32, device=q.device)
    rc = _lib.lib().mcb_dsa_index_scores(_lib.ptr(q.contiguous()), _lib.ptr(k.contiguous()),
                                         _lib.ptr(w.float().contiguous()), _lib.ptr(seq_start), _lib.ptr(out),
                                         ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(D),
                                         _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_dsa_index_scores')
    return out


def topk_indices(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Positions of the ``k`` largest entries of every row (unordered), radix-select kernel on CUDA."""
    import ctypes

    from . import _lib
    if not (scores.is_cuda and scores.dtype == torch.float32 and scores.dim() == 2 and _lib.available()):
        return scores.topk(k, dim=-1).indices
    rows, n = scores.shape
    s = scores if scores.stride(1) == 1 else scores.contiguous()
    idx = torch.empty((rows, k), dtype=torch.int64, device=scores.device)
    rc = _lib.lib().mcb_topk_select(_lib.ptr(s), ctypes.c_longlong(s.stride(0)), ctypes.c_int(rows), ctypes.c_int(n),
                                    ctypes.c_int(k), _lib.ptr(idx), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_topk_select')
    return idx


# ------------------------------------------------------------------------------------------------ scalable path
def sparse_mla_attention_absorbed(q_nope: torch.Tensor, q_pe: torch.Tensor, kv_lat: torch.Tensor, k_pe: torch.Tensor,
                                  w_uk: torch.Tensor, w_uv: torch.Tensor, idx: torch.Tensor, seq_start: torch.Tensor,
                                  scale: float, chunk: int = 512) -> torch.Tensor:
    """Top-k sparse MLA attention in the weight-absorbed (latent, multi-query) form, one block of queries at a time.

    ``q_nope [T, h, dn]``, ``q_pe [T, h, dr]`` (rotated), ``kv_lat [T, dl]`` (normalised latent), ``k_pe [T, dr]``
    (rotated, shared by the heads), ``w_uk [h, dn, dl]`` / ``w_uv [h, dv, dl]`` (the two halves of the kv
    up-projection),
    ``idx [T, topk]`` selected key positions, ``seq_start [T]``.  Scores are ``(q_nope W_uk) . c_kv + q_pe . k_pe`` over
    the selected keys only, so memory is ``O(chunk * topk)`` instead of ``O(T^2)`` and the work is the sparse work.  A
    selected position that the query may not see (later than the query or in another sequence: rows with fewer than
    top-k visible keys) is masked.  Each block runs under activation checkpointing: its gathered keys are rebuilt in
    backward, not stored.  Equal to :func:`sparse_attention` on the explicit per-head keys / values.
    """
    from torch.utils.checkpoint import checkpoint
    T, h, dn = q_nope.shape
    dv = w_uv.shape[1]
    q_abs = torch.einsum('thn,hnl->thl', q_nope, w_uk.to(q_nope.dtype))                     # [T, h, dl]

    def block(qa, qp, ids, lo, pos, lat, kpe):
        sel = lat[ids]                                                                      # [C, K, dl]
        pe = kpe[ids]                                                                       # [C, K, dr]
        s = torch.einsum('chl,ckl->chk', qa, sel).float() + torch.einsum('chr,ckr->chk', qp, pe).float()
        s = s * scale
        vis = (ids <= pos[:, None]) & (ids >= lo[:, None])                                  # [C, K]
        s = s.masked_fill(~vis[:, None, :], float('-inf'))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0).to(sel.dtype)
        return torch.einsum('chk,ckl->chl', p, sel)                                         # [C, h, dl]

    outs = []
    pos_all = torch.arange(T, device=q_nope.device)
    lo_all = seq_start.to(torch.int64)
    for c0 in range(0, T, chunk):
        c1 = min(T, c0 + chunk)
        args = (q_abs[c0:c1], q_pe[c0:c1], idx[c0:c1], lo_all[c0:c1], pos_all[c0:c1], kv_lat, k_pe)
        if torch.is_grad_enabled() and (q_nope.requires_grad or kv_lat.requires_grad):
            outs.append(checkpoint(block, *args, use_reentrant=False))
        else:
            outs.append(block(*args))
    o_lat = torch.cat(outs, dim=0)
    return torch.einsum('thl,hvl->thv', o_lat, w_uv.to(o_lat.dtype)).contiguous()
