"""Variable-length (packed) causal attention with GQA, sliding window and learnable softmax sinks.

Inputs are token-major: ``q [T, nq, d]``, ``k [T, nkv, d]``, ``v [T, nkv, dv]`` plus ``cu_seqlens``
(int32 ``[B+1]``) delimiting the packed sequences; tokens never attend across a boundary.

On a GPU the in-tree sm_100a kernel (``csrc/attention``) runs every configuration it covers.  A configuration it
does not cover is handed to the ``flash_attn`` library kernel (or, for what that lacks too, the masked-softmax
reference) with a warning logged once per kind of gap, so a model that leaves the in-tree path says so;
``MCB200_ATTENTION_BACKEND=mcb`` turns that into an error.  On CPU the masked fp32 softmax is the oracle.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch


def segment_ids(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """``[T]`` index of the packed sequence each token belongs to."""
    pos = torch.arange(total, device=cu_seqlens.device)
    return torch.searchsorted(cu_seqlens[1:].to(torch.int64).contiguous(), pos, right=True)


def attention_ref(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, causal=True, scale=None,
                  window: Optional[Tuple[int, int]] = None, sinks: Optional[torch.Tensor] = None,
                  softcap: Optional[float] = None, q_pos: Optional[torch.Tensor] = None,
                  k_pos: Optional[torch.Tensor] = None, return_lse: bool = False):
    """fp32 masked softmax attention.  ``q_pos``/``k_pos`` (positions inside each sequence) allow query and
    key sets that are not aligned suffixes (context parallel chunks); default is position = index in sequence."""
    Tq, nq, d = q.shape
    Tk, nkv, dv = v.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    dev = q.device
    if cu_seqlens_q is None:
        cu_seqlens_q = torch.tensor([0, Tq], dtype=torch.int32, device=dev)
    if cu_seqlens_k is None:
        cu_seqlens_k = cu_seqlens_q if Tk == Tq else torch.tensor([0, Tk], dtype=torch.int32, device=dev)
    sq, sk = segment_ids(cu_seqlens_q, Tq), segment_ids(cu_seqlens_k, Tk)
    if q_pos is None:
        # align the ends of q and k inside each sequence (standard bottom-right causal alignment)
        lq = (cu_seqlens_q[1:] - cu_seqlens_q[:-1]).to(torch.int64)
        lk = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).to(torch.int64)
        q_pos = torch.arange(Tq, device=dev) - cu_seqlens_q[:-1].to(torch.int64)[sq] + (lk - lq)[sq]
    if k_pos is None:
        k_pos = torch.arange(Tk, device=dev) - cu_seqlens_k[:-1].to(torch.int64)[sk]
    mask = sq[:, None] == sk[None, :]
    if causal:
        mask = mask & (k_pos[None, :] <= q_pos[:, None])
    if window is not None and window[0] is not None and window[0] >= 0:
        mask = mask & (q_pos[:, None] - k_pos[None, :] <= window[0])
    if window is not None and len(window) > 1 and window[1] is not None and window[1] >= 0 and not causal:
        mask = mask & (k_pos[None, :] - q_pos[:, None] <= window[1])
    rep = nq // nkv
    qf = q.float().transpose(0, 1)                                  # [nq, Tq, d]
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)    # [nq, Tk, d]
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~mask[None], float('-inf'))
    if sinks is not None:
        s = torch.cat([s, sinks.float().view(nq, 1, 1).expand(nq, Tq, 1)], dim=-1)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)   # rows with no visible key
    if sinks is not None:
        p = p[..., :-1]
    o = torch.matmul(p, vf).transpose(0, 1).to(q.dtype).contiguous()
    if return_lse:
        return o, lse
    return o


def _flash_attn_available() -> bool:
    try:
        import flash_attn  # noqa: F401
        return True
    except Exception:
        return False


_BACKEND_ENV = 'MCB200_ATTENTION_BACKEND'  # auto | mcb | flash_attn | torch


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None,
              max_seqlen: Optional[int] = None, causal: bool = True, scale: Optional[float] = None,
              window: Optional[Tuple[int, int]] = None, sinks: Optional[torch.Tensor] = None,
              softcap: Optional[float] = None, seq_start: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Self-attention over packed sequences; returns ``[T, nq, dv]``.  ``seq_start`` (``[T]`` int32, first token
    of each token's sequence) can be passed to avoid recomputing it in every layer."""
    backend = os.environ.get(_BACKEND_ENV, 'auto')
    T, nq, d = q.shape
    if q.is_cuda and backend in ('auto', 'mcb'):
        from . import _lib, attention_cuda
        why = attention_cuda.unsupported_reason(q, k, v, causal, window, sinks, softcap)
        if why is None and _lib.available():
            return attention_cuda.attention(q, k, v, cu_seqlens, max_seqlen, scale, seq_start, window, sinks)
        if backend == 'mcb':
            raise RuntimeError('the in-tree attention kernel does not cover '
                               f'{why or "a run with the kernels disabled"}')
        if why is not None and _lib.cuda_enabled():
            from ..utils.logger import get_logger
            get_logger().warning_once(f'attention: the in-tree sm_100a kernel does not cover {why}; '
                                      'this call runs on a library / reference kernel')
    if q.is_cuda and backend in ('auto', 'flash_attn') and sinks is None \
            and q.dtype in (torch.bfloat16, torch.float16) and _flash_attn_available() and d <= 256:
        from flash_attn import flash_attn_varlen_func
        if cu_seqlens is None:
            cu_seqlens = torch.tensor([0, T], dtype=torch.int32, device=q.device)
            max_seqlen = T
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
        ws = (-1, -1) if window is None else (int(window[0]), 0 if causal else int(window[1]))
        vv = v
        if v.shape[-1] != d:  # MLA: value head narrower than qk head
            vv = torch.nn.functional.pad(v, (0, d - v.shape[-1]))
        o = flash_attn_varlen_func(q, k, vv, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, softmax_scale=scale,
                                   causal=causal, window_size=ws, softcap=softcap or 0.0)
        return o[..., :v.shape[-1]] if v.shape[-1] != d else o
    return attention_ref(q, k, v, cu_seqlens, cu_seqlens, causal, scale, window, sinks, softcap)


def attention_qk_ranges(q: torch.Tensor, k_full: torch.Tensor, v_full: torch.Tensor, lay, scale=None, window=None,
                        sinks=None) -> torch.Tensor:
    """Attention of a context-parallel rank's queries ``[T_local, nq, d]`` against the keys / values of the whole
    token stream (``lay`` = ``parallel.context_parallel.CpLayout``), for what the in-tree ranges kernel does not
    cover: the masked-softmax reference with explicit positions (memory O(T_local x T): meant for CPU tests and
    small inputs)."""
    k_rel = torch.arange(k_full.shape[0], device=q.device) - \
        lay.cu_full.to(torch.int64)[segment_ids(lay.cu_full, k_full.shape[0])]
    return attention_ref(q, k_full, v_full, lay.cu_local, lay.cu_full, True, scale, window, sinks, None, lay.q_rel,
                         k_rel)
