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


def index_scores(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, mask: torch.Tensor, chunk: int = 2048) -> torch.Tensor:
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
                    idx: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``scores [T, Tk]`` (with ``-inf`` outside the mask), ``attn_probs [h, T, Tk]`` -> scalar KL."""
    target = attn_probs.sum(0)
    keep = mask if idx is None else (topk_mask(idx, scores.shape[1]) & mask)
    target = target.masked_fill(~keep, 0.0)
    target = target / target.sum(-1, keepdim=True).clamp(min=1e-20)
    logp = torch.log_softmax(scores.masked_fill(~keep, float('-inf')), dim=-1)
    logp = torch.where(keep, logp, torch.zeros_like(logp))
    kl = (target * (torch.log(target.clamp(min=1e-20)) - logp)).sum(-1)
    return kl.mean()
