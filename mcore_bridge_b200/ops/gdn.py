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

import functools
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def _bounds(cu_seqlens: Optional[torch.Tensor], T: int) -> List[Tuple[int, int]]:
    if cu_seqlens is None:
        return [(0, T)]
    from ..utils.torch_utils import host_list
    b = host_list(cu_seqlens)
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
        k_dec = k[:, i] * (g_last[:, None] - gc[:, i]).exp()[..., None]
        S = S * g_last.exp()[:, None, None] + k_dec.transpose(-1, -2) @ v_new
    return torch.stack(outs, dim=1).reshape(h, n * chunk, dv)[:, :L]


class _ChunkPlan:
    """Host-side layout of a packed batch for the chunked rule, with its index tensors on the device."""
    __slots__ = ('total', 'n_seq', 'tok_idx', 'slot_idx', 'first', 'alive', 'identity')


@functools.lru_cache(maxsize=16)
def _chunk_plan(bounds: Tuple[Tuple[int, int], ...], T: int, chunk: int, device: str) -> _ChunkPlan:
    """Sequences sorted by length (longest first) and padded to whole chunks: token -> slot indices, first chunk of
    every sequence, and how many sequences are still running at every chunk position.  Sorting makes "the sequences
    still running" a prefix, so the recurrence slices instead of asking the device which ones are left; the plan is
    cached because every layer of a step sees the same batch."""
    dev = torch.device(device)
    order = sorted(range(len(bounds)), key=lambda j: -(bounds[j][1] - bounds[j][0]))
    tok, slot, first, counts, off = [], [], [], [], 0
    for j in order:
        s, e = bounds[j]
        n = -(-(e - s) // chunk)
        tok.append(torch.arange(s, e))
        slot.append(torch.arange(off * chunk, off * chunk + (e - s)))
        first.append(off)
        counts.append(n)
        off += n
    p = _ChunkPlan()
    p.total, p.n_seq = off, len(order)
    tok_idx = torch.cat(tok) if tok else torch.zeros(0, dtype=torch.int64)
    slot_idx = torch.cat(slot) if slot else torch.zeros(0, dtype=torch.int64)
    p.identity = tok_idx.numel() == T == off * chunk and bool((tok_idx == slot_idx).all())
    p.tok_idx, p.slot_idx = tok_idx.to(dev), slot_idx.to(dev)
    p.first = torch.tensor(first, dtype=torch.int64).to(dev)
    p.alive = tuple(sum(1 for n in counts if n > i) for i in range(max(counts) if counts else 0))
    return p


def chunk_gated_delta_rule(q, k, v, g, beta, cu_seqlens=None, scale: Optional[float] = None, chunk: int = 64):
    """Chunked evaluation; same signature and result as :func:`recurrent_gated_delta_rule`.

    All sequences are processed together: every sequence is padded to a whole number of chunks, the intra-chunk
    quantities (decay matrix, WY solve, intra-chunk attention) are one batched computation over all chunks, and the
    state recurrence runs over the chunk *position inside its sequence*, i.e. ``max_len / chunk`` steps of batched
    matmuls over the sequences still running, rather than one step per chunk of the packed stream.  Apart from reading
    the sequence boundaries, nothing in here waits for the device."""
    T, h, dk = q.shape
    dv = v.shape[-1]
    dev = q.device
    scale = dk**-0.5 if scale is None else scale
    plan = _chunk_plan(tuple(_bounds(cu_seqlens, T)), T, chunk, str(dev))
    total = plan.total

    def pad(x):
        if plan.identity:
            return x.float()
        out = x.new_zeros((total * chunk, *x.shape[1:]), dtype=torch.float32)
        return out.index_copy(0, plan.slot_idx, x.float().index_select(0, plan.tok_idx))

    qp = (pad(q) * scale).view(total, chunk, h, dk).permute(0, 2, 1, 3)          # [N, h, C, dk]
    kp = pad(k).view(total, chunk, h, dk).permute(0, 2, 1, 3)
    vp = pad(v).view(total, chunk, h, dv).permute(0, 2, 1, 3)
    gp = pad(g).view(total, chunk, h).permute(0, 2, 1)                            # [N, h, C]
    bp = pad(beta).view(total, chunk, h).permute(0, 2, 1)
    gc = gp.cumsum(-1)
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()
    kb, vb = kp * bp[..., None], vp * bp[..., None]
    eye = torch.eye(chunk, dtype=torch.float32, device=dev)
    A = eye + ((kb @ kp.transpose(-1, -2)) * decay).tril(-1)
    u = torch.linalg.solve_triangular(A, vb, upper=False, unitriangular=True)
    w = torch.linalg.solve_triangular(A, kb * gc.exp()[..., None], upper=False, unitriangular=True)
    qk = (qp @ kp.transpose(-1, -2)) * decay
    q_dec = qp * gc.exp()[..., None]
    g_last = gc[..., -1]                                                          # [N, h]
    k_dec = kp * (g_last[..., None] - gc).exp()[..., None]
    S = torch.zeros(plan.n_seq, h, dk, dv, dtype=torch.float32, device=dev)
    outs, ids = [], []
    for i, m in enumerate(plan.alive):
        ci = plan.first[:m] + i                                                   # chunk ids processed this step
        Si = S[:m]
        v_new = u[ci] - w[ci] @ Si
        outs.append(q_dec[ci] @ Si + qk[ci] @ v_new)
        ids.append(ci)
        S = Si * g_last[ci].exp()[..., None, None] + k_dec[ci].transpose(-1, -2) @ v_new
    out = torch.zeros(total, h, chunk, dv, dtype=torch.float32, device=dev)
    if outs:
        out = out.index_copy(0, torch.cat(ids), torch.cat(outs))
    o_flat = out.permute(0, 2, 1, 3).reshape(total * chunk, h, dv)
    if plan.identity:
        return o_flat.to(v.dtype)
    res = torch.zeros(T, h, dv, dtype=torch.float32, device=dev)
    return res.index_copy(0, plan.tok_idx, o_flat.index_select(0, plan.slot_idx)).to(v.dtype)


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


# ------------------------------------------------------------------------------------------------ simple GLA
def simple_gla_ref(q, k, v, decay, cu_seqlens=None, scale: Optional[float] = None) -> torch.Tensor:
    """Linear attention with a constant per-head log-decay ``decay [h] <= 0``::

        S_t = exp(decay_h) * S_{t-1} + k_t v_t^T,      o_t = scale * S_t^T q_t

    evaluated per sequence as ``(Q K^T * D) V`` with ``D[i, j] = exp(decay * (i - j))`` for ``j <= i`` (fp32).  The
    recurrence the reference runs through fla's ``fused_recurrent_simple_gla``
    (``src/mcore_bridge/model/gpts/bailing_hybrid.py:180-193``)."""
    T, h, dk = q.shape
    scale = dk**-0.5 if scale is None else scale
    out = torch.empty(T, h, v.shape[-1], dtype=torch.float32, device=q.device)
    for s, e in _bounds(cu_seqlens, T):
        L = e - s
        pos = torch.arange(L, device=q.device, dtype=torch.float32)
        diff = pos[:, None] - pos[None, :]
        D = torch.exp(decay.float()[:, None, None] * diff.clamp(min=0)[None]) * (diff >= 0)[None]
        att = torch.einsum('ihd,jhd->hij', q[s:e].float() * scale, k[s:e].float()) * D
        out[s:e] = torch.einsum('hij,jhd->ihd', att, v[s:e].float())
    return out.to(v.dtype)


# ------------------------------------------------------------------------------------------------ CUDA dispatch
def _cuda_ok(*ts) -> bool:
    from . import _lib
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and _lib.available()


def _seq_start(cu_seqlens, T, device):
    from .attention_cuda import seq_start_from_cu
    return seq_start_from_cu(cu_seqlens, T, device)


class _ConvFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, seq_start, act):
        import ctypes

        from . import _lib
        T, C = x.shape
        x, w = x.contiguous(), weight.contiguous()
        y = torch.empty_like(x)
        rc = _lib.lib().mcb_conv1d_silu_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(seq_start), _lib.ptr(y), ctypes.c_int(T),
                                            ctypes.c_int(C), ctypes.c_int(w.shape[1]), ctypes.c_int(int(act)),
                                            _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_conv1d_silu_fwd')
        ctx.save_for_backward(x, w, seq_start)
        ctx.act = act
        return y

    @staticmethod
    def backward(ctx, dy):
        import ctypes

        from . import _lib
        x, w, seq_start = ctx.saved_tensors
        T, C = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
        rc = _lib.lib().mcb_conv1d_silu_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(seq_start), _lib.ptr(dx),
                                            _lib.ptr(dw), ctypes.c_int(T), ctypes.c_int(C), ctypes.c_int(w.shape[1]),
                                            ctypes.c_int(int(ctx.act)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_conv1d_silu_bwd')
        return dx, dw.to(w.dtype), None, None


class _GatedNormFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        import ctypes

        from . import _lib
        D = x.shape[-1]
        x2, z2, w = x.reshape(-1, D).contiguous(), gate.reshape(-1, D).contiguous(), weight.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _lib.lib().mcb_gated_rmsnorm_fwd(_lib.ptr(x2), _lib.ptr(z2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd),
                                              ctypes.c_longlong(rows), ctypes.c_int(D), ctypes.c_float(eps),
                                              _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_gated_rmsnorm_fwd')
        ctx.save_for_backward(x2, z2, w, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        import ctypes

        from . import _lib
        x2, z2, w, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = dy.reshape(rows, D).contiguous()
        dx, dz = torch.empty_like(x2), torch.empty_like(z2)
        dw = torch.zeros(D, dtype=torch.float32, device=x2.device)
        rc = _lib.lib().mcb_gated_rmsnorm_bwd(_lib.ptr(x2), _lib.ptr(z2), _lib.ptr(w), _lib.ptr(dy2), _lib.ptr(rstd),
                                              _lib.ptr(dx), _lib.ptr(dz), _lib.ptr(dw), ctypes.c_longlong(rows),
                                              ctypes.c_int(D), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_gated_rmsnorm_bwd')
        return dx.view(ctx.shape), dz.view(ctx.shape), dw.to(w.dtype), None


class _SimpleGlaFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, decay, cu_seqlens, scale):
        import ctypes

        from . import _lib
        T, h, dk = q.shape
        dv = v.shape[-1]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        decay = decay.float().contiguous()
        o = torch.empty_like(v)
        n_seq = cu_seqlens.numel() - 1
        rc = _lib.lib().mcb_simple_gla_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(decay), _lib.ptr(cu_seqlens),
                                           _lib.ptr(o), ctypes.c_int(n_seq), ctypes.c_int(h), ctypes.c_int(dk),
                                           ctypes.c_int(dv), ctypes.c_float(scale), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_simple_gla_fwd')
        ctx.save_for_backward(q, k, v, decay, cu_seqlens)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        import ctypes

        from . import _lib
        q, k, v, decay, cu = ctx.saved_tensors
        T, h, dk = q.shape
        dv_ = v.shape[-1]
        do = do.contiguous()
        dq, dk_, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        rc = _lib.lib().mcb_simple_gla_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(do), _lib.ptr(decay),
                                           _lib.ptr(cu), _lib.ptr(dq), _lib.ptr(dk_), _lib.ptr(dv),
                                           ctypes.c_int(cu.numel() - 1), ctypes.c_int(h), ctypes.c_int(dk),
                                           ctypes.c_int(dv_), ctypes.c_float(ctx.scale), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_simple_gla_bwd')
        return dq, dk_, dv, None, None, None


def simple_gla(q, k, v, decay, cu_seqlens=None, scale: Optional[float] = None) -> torch.Tensor:
    """Dispatches to the recurrent CUDA kernels (bf16, square 64 / 128 state) or the torch restatement."""
    T, h, dk = q.shape
    scale = dk**-0.5 if scale is None else scale
    if _cuda_ok(q, k, v) and dk == v.shape[-1] and dk in (64, 128):
        cu = cu_seqlens if cu_seqlens is not None else torch.tensor([0, T], dtype=torch.int32, device=q.device)
        return _SimpleGlaFn.apply(q, k, v, decay, cu.to(device=q.device, dtype=torch.int32), float(scale))
    return simple_gla_ref(q, k, v, decay, cu_seqlens, scale)


_causal_conv1d_silu_torch = causal_conv1d_silu
_gated_rmsnorm_torch = gated_rmsnorm


def causal_conv1d_silu(x, weight, bias=None, cu_seqlens=None, activation: bool = True, seq_start=None):  # noqa: F811
    if bias is None and _cuda_ok(x, weight) and x.shape[1] % 8 == 0 and weight.shape[-1] in (2, 3, 4):
        if seq_start is None:
            seq_start = _seq_start(cu_seqlens, x.shape[0], x.device)
        return _ConvFn.apply(x, weight, seq_start, bool(activation))
    return _causal_conv1d_silu_torch(x, weight, bias, cu_seqlens, activation)


def gated_rmsnorm(x, gate, weight, eps):  # noqa: F811
    if _cuda_ok(x, gate, weight) and x.shape[-1] in (64, 128, 256):
        return _GatedNormFn.apply(x, gate, weight, float(eps))
    return _gated_rmsnorm_torch(x, gate, weight, eps)
