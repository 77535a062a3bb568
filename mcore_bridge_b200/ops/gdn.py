"""Gated delta rule (the linear-attention core of Qwen3-Next's gated DeltaNet), causal depthwise conv1d + SiLU,
gated RMSNorm.  Torch implementations; they are the oracle for the CUDA kernels and the CPU path.

Recurrence per head, state ``S [dk, dv]``, decay ``g_t <= 0``, write strength ``beta_t``::

    S   <- exp(g_t) * S
    S   <- S + beta_t * k_t (v_t - S^T k_t)^T
    o_t  = S^T q_t

:func:`chunk_gated_delta_rule` evaluates it chunk-wise (64 tokens): inside a chunk the rank-1 updates are
resolved with one unit-lower-triangular solve (WY form), between chunks only the state is carried.
:func:`recurrent_gated_delta_rule` is the token-by-token definition used to test it.  Both accept packed
sequences through ``cu_seqlens`` (the state is reset at every boundary).  Numerics (fp32 cumulative decays) match
Transformers' ``torch_chunk_gated_delta_rule`` (``modeling_qwen3_next.py``) and the reference's call at
``src/mcore_bridge/model/modules/gated_delta_net.py:328-351``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def _bounds(cu_seqlens: Optional[torch.Tensor], T: int) -> List[Tuple[int, int]]:
    if cu_seqlens is None:
        return [(0, T)]
    b = [int(x) for x in cu_seqlens.tolist()]
    return [(s, e) for s, e in zip(b[:-1], b[1:]) if e > s]


def recurrent_gated_delta_rule(q, k, v, g, beta, cu_seqlens=None, scale: Optional[float] = None) -> torch.Tensor:
    """``q, k [T, h, dk]``, ``v [T, h, dv]``, ``g, beta [T, h]`` -> ``o [T, h, dv]`` (fp32 math)."""
    T, h, dk = q.shape
    dv = v.shape[-1]
    scale = dk**-0.5 if scale is None else scale
    qf, kf, vf, gf, bf = q.float() * scale, k.float(), v.float(), g.float(), beta.float()
    out = torch.zeros(T, h, dv, dtype=torch.float32, device=q.device)
    for s, e in _bounds(cu_seqlens, T):
        S = torch.zeros(h, dk, dv, dtype=torch.float32, device=q.device)
        for t in range(s, e):
            S = S * gf[t].exp()[:, None, None]
            mem = torch.einsum('hkv,hk->hv', S, kf[t])
            delta = (vf[t] - mem) * bf[t][:, None]
            S = S + kf[t][:, :, None] * delta[:, None, :]
            out[t] = torch.einsum('hkv,hk->hv', S, qf[t])
    return out.to(v.dtype)


def _chunk_one_sequence(q, k, v, g, beta, chunk: int):
    """One sequence, tensors ``[h, L, d]`` fp32 (already scaled); returns ``[h, L, dv]``."""
    h, L, dk = q.shape
    dv = v.shape[-1]
    pad = (-L) % chunk
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, pad)) for x in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    n = (L + pad) // chunk
    q, k, v = (x.reshape(h, n, chunk, -1) for x in (q, k, v))
    g, beta = g.reshape(h, n, chunk), beta.reshape(h, n, chunk)
    gc = g.cumsum(-1)                                               # cumulative log-decay inside the chunk
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()   # [h, n, C, C], lower incl. diagonal
    kb, vb = k * beta[..., None], v * beta[..., None]
    L_mat = (kb @ k.transpose(-1, -2)) * decay
    eye = torch.eye(chunk, dtype=q.dtype, device=q.device)
    A = eye + L_mat.tril(-1)                                        # unit lower triangular
    u = torch.linalg.solve_triangular(A, vb, upper=False, unitriangular=True)                   # pseudo-values
    w = torch.linalg.solve_triangular(A, kb * gc.exp()[..., None], upper=False, unitriangular=True)
    S = torch.zeros(h, dk, dv, dtype=q.dtype, device=q.device)
    outs = []
    qk = (q @ k.transpose(-1, -2)) * decay                          # intra-chunk attention (causal incl. diagonal)
    for i in range(n):
        v_new = u[:, i] - w[:, i] @ S                               # [h, C, dv]
        o = (q[:, i] * gc[:, i].exp()[..., None]) @ S + qk[:, i] @ v_new
        outs.append(o)
        g_last = gc[:, i, -1]
        S = S * g_last.exp()[:, None, None] + (k[:, i] * (g_last[:, None] - gc[:, i]).exp()[..., None]).transpose(-1, -2) @ v_new
    return torch.stack(outs, dim=1).reshape(h, n * chunk, dv)[:, :L]


def chunk_gated_delta_rule(q, k, v, g, beta, cu_seqlens=None, scale: Optional[float] = None, chunk: int = 64):
    """Chunked evaluation; same signature and result as :func:`recurrent_gated_delta_rule`."""
    T, h, dk = q.shape
    scale = dk**-0.5 if scale is None else scale
    qf = (q.float() * scale).transpose(0, 1)
    kf, vf = k.float().transpose(0, 1), v.float().transpose(0, 1)
    gf, bf = g.float().transpose(0, 1), beta.float().transpose(0, 1)
    outs = []
    for s, e in _bounds(cu_seqlens, T):
        outs.append(_chunk_one_sequence(qf[:, s:e], kf[:, s:e], vf[:, s:e], gf[:, s:e], bf[:, s:e], chunk))
    return torch.cat(outs, dim=1).transpose(0, 1).to(v.dtype)


def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       cu_seqlens: Optional[torch.Tensor] = None, activation: bool = True) -> torch.Tensor:
    """Depthwise causal convolution over tokens: ``x [T, C]``, ``weight [C, K]``; every packed sequence starts
    from zero history.  ``y[t, c] = sum_j w[c, j] * x[t - (K-1) + j, c]``, then SiLU."""
    T, C = x.shape
    K = weight.shape[-1]
    outs = []
    for s, e in _bounds(cu_seqlens, T):
        xs = x[s:e].transpose(0, 1).unsqueeze(0)                    # [1, C, L]
        y = F.conv1d(xs, weight.unsqueeze(1).to(x.dtype), None if bias is None else bias.to(x.dtype), padding=K - 1,
                     groups=C)[..., :e - s]
        outs.append(y.squeeze(0).transpose(0, 1))
    y = torch.cat(outs, dim=0)
    return F.silu(y) if activation else y


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``rmsnorm(x) * weight * silu(gate)`` over the last dim (norm before gate)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = weight.float() * y.to(x.dtype).float()
    return (y * F.silu(gate.float())).to(x.dtype)
