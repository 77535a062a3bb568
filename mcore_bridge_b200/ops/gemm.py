"""bf16 GEMM on the tcgen05 tile engine (``csrc/gemm``), with a torch fallback for CPU runs.

Three layouts cover a linear layer without transposed copies:

* :func:`mm_nt`  ``y[M,N] = x[M,K] @ w[N,K]^T``      forward
* :func:`mm_nn`  ``dx[M,K] = dy[M,N] @ w[N,K]``       input gradient
* :func:`mm_tn`  ``dw[N,K] = dy[T,N]^T @ x[T,K]``     weight gradient (optionally accumulated in fp32)

and the grouped variants (:func:`grouped_mm_nt`, :func:`grouped_mm_nn`, :func:`grouped_mm_tn`) run every
expert of an MoE layer in one persistent launch with device-resident group offsets.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib

DENSE, GROUPED_M, GROUPED_K = 0, 1, 2
_c_ll = ctypes.c_longlong
_c_int = ctypes.c_int


def _use_cuda(*ts) -> bool:
    return all(t is None or t.is_cuda for t in ts) and ts[0].dtype == torch.bfloat16 and _lib.available()


def _launch(a, a_inner, a_outer, lda, a_mn, b, b_inner, b_outer, ldb, b_mn, c, ldc, c_group_stride, M, N, K, alpha,
            bias, accumulate, mode=DENSE, num_groups=0, offsets=None, b_group_rows=0, max_sms=0, force_bn=0):
    rc = _lib.lib().mcb_gemm_bf16(
        _lib.ptr(a), _c_ll(a_inner), _c_ll(a_outer), _c_ll(lda), _c_int(int(a_mn)),
        _lib.ptr(b), _c_ll(b_inner), _c_ll(b_outer), _c_ll(ldb), _c_int(int(b_mn)),
        _lib.ptr(c), _c_ll(ldc), _c_ll(c_group_stride), _c_int(int(c.dtype == torch.float32)), _c_int(int(accumulate)),
        _c_int(M), _c_int(N), _c_int(K), ctypes.c_float(alpha), _lib.ptr(bias),
        _c_int(mode), _c_int(num_groups), _lib.ptr(offsets), _c_int(b_group_rows),
        _lib.ptr(_lib.status_word(a.device)), _c_int(max_sms), _c_int(force_bn), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_gemm_bf16')


def _lib_mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b`` for the paths without the in-tree kernels, returned in fp32.  On the CPU (the oracle of the tests) the
    product is formed in fp32; on a GPU with the kernels switched off it is the library's GEMM in the operands' own
    dtype (bf16 inputs, fp32 accumulation), which is what a stack built on cuBLAS would run."""
    if a.is_cuda and a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16):
        return torch.matmul(a, b).float()
    return torch.matmul(a.float(), b.float())


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    """Returns a 2-D view whose last dim is contiguous and whose row stride is TMA-compatible."""
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def _out(out, shape, dtype, device, accumulate):
    if out is None:
        assert not accumulate, 'accumulate needs an output tensor'
        return torch.empty(shape, dtype=dtype, device=device)
    assert tuple(out.shape) == tuple(shape) and out.stride(-1) == 1, (out.shape, shape, out.stride())
    return out


def mm_nt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
          out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
          max_sms: int = 0, force_bn: int = 0) -> torch.Tensor:
    """``x[..., K] @ w[N, K]^T (+ bias)``."""
    lead = x.shape[:-1]
    K = x.shape[-1]
    N = w.shape[0]
    assert w.shape[1] == K
    if not _use_cuda(x, w, bias):
        y = _lib_mm(x.reshape(-1, K), w.t()) * alpha
        if bias is not None:
            y = y + bias.float()
        y = y.to(out_dtype or x.dtype)
        if out is not None:
            if accumulate:
                out.add_(y.view(out.shape))
            else:
                out.copy_(y.view(out.shape))
            return out
        return y if len(lead) == 1 else y.view(*lead, N)
    x2, w2 = _row_major_2d(x), _row_major_2d(w)
    M = x2.shape[0]
    c = _out(out.view(M, N) if out is not None else None, (M, N), out_dtype or torch.bfloat16, x.device, accumulate)
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    _launch(x2, K, M, x2.stride(0), False, w2, K, N, w2.stride(0), False, c, c.stride(0), 0, M, N, K, alpha, bias,
            accumulate, max_sms=max_sms, force_bn=force_bn)
    if out is not None:
        return out
    return c if len(lead) == 1 else c.view(*lead, N)      # no alias for the common 2-D case: callers may add in place


def mm_nn(dy: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
          out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
          max_sms: int = 0, force_bn: int = 0) -> torch.Tensor:
    """``dy[..., N] @ w[N, K]`` -> ``[..., K]``."""
    lead = dy.shape[:-1]
    N = dy.shape[-1]
    K = w.shape[1]
    assert w.shape[0] == N
    if not _use_cuda(dy, w):
        y = (_lib_mm(dy.reshape(-1, N), w) * alpha).to(out_dtype or dy.dtype)
        if out is not None:
            if accumulate:
                out.add_(y.view(out.shape))
            else:
                out.copy_(y.view(out.shape))
            return out
        return y if len(lead) == 1 else y.view(*lead, K)
    d2, w2 = _row_major_2d(dy), _row_major_2d(w)
    M = d2.shape[0]
    c = _out(out.view(M, K) if out is not None else None, (M, K), out_dtype or torch.bfloat16, dy.device, accumulate)
    # A = dy (K-major over the contraction N); B[k_out, n] = w[n, k_out] is MN-major as stored
    _launch(d2, N, M, d2.stride(0), False, w2, K, N, w2.stride(0), True, c, c.stride(0), 0, M, K, N, alpha, None,
            accumulate, max_sms=max_sms, force_bn=force_bn)
    if out is not None:
        return out
    return c if len(lead) == 1 else c.view(*lead, K)


def mm_tn(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None,
          out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
          max_sms: int = 0, force_bn: int = 0) -> torch.Tensor:
    """``dy[T, N]^T @ x[T, K]`` -> ``[N, K]`` (weight gradient)."""
    N = dy.shape[-1]
    K = x.shape[-1]
    if not _use_cuda(dy, x):
        y = (_lib_mm(dy.reshape(-1, N).t(), x.reshape(-1, K)) * alpha)
        if out is not None:
            if accumulate:
                out.add_(y.to(out.dtype))
            else:
                out.copy_(y.to(out.dtype))
            return out
        return y.to(out_dtype or dy.dtype)
    d2, x2 = _row_major_2d(dy), _row_major_2d(x)
    T = d2.shape[0]
    assert x2.shape[0] == T
    c = _out(out, (N, K), out_dtype or torch.bfloat16, dy.device, accumulate)
    _launch(d2, N, T, d2.stride(0), True, x2, K, T, x2.stride(0), True, c, c.stride(0), 0, N, K, T, alpha, None,
            accumulate, max_sms=max_sms, force_bn=force_bn)
    return c


# ------------------------------------------------------------------ grouped (MoE experts)
def _check_offsets(offsets: torch.Tensor):
    assert offsets.dtype == torch.int32 and offsets.dim() == 1


def grouped_mm_nt(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[r] = x[r] @ w[g(r)]^T`` for rows grouped by expert.

    ``x`` is ``[R, K]`` with group ``g`` owning rows ``offsets[g]:offsets[g+1]`` (every offset a multiple of
    128; rows past ``offsets[-1]`` are ignored), ``w`` is ``[G, N, K]``.
    """
    _check_offsets(offsets)
    G, N, K = w.shape
    R = x.shape[0]
    if not _use_cuda(x, w, offsets):
        y = torch.zeros(R, N, dtype=x.dtype, device=x.device) if out is None else out
        off = offsets.tolist()
        for g in range(G):
            s, e = off[g], off[g + 1]
            if e > s:
                r = _lib_mm(x[s:e], w[g].t())
                if bias is not None:
                    r = r + bias[g].float()
                y[s:e] = r.to(y.dtype)
        return y
    x2 = _row_major_2d(x)
    w2 = w.contiguous().view(G * N, K)
    c = _out(out, (R, N), torch.bfloat16, x.device, False)
    _launch(x2, K, R, x2.stride(0), False, w2, K, G * N, K, False, c, c.stride(0), 0, R, N, K, 1.0, bias, False,
            mode=GROUPED_M, num_groups=G, offsets=offsets, b_group_rows=N)
    return c


def grouped_mm_nn(dy: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dx[r] = dy[r] @ w[g(r)]`` with ``dy [R, N]``, ``w [G, N, K]`` -> ``[R, K]``."""
    _check_offsets(offsets)
    G, N, K = w.shape
    R = dy.shape[0]
    if not _use_cuda(dy, w, offsets):
        y = torch.zeros(R, K, dtype=dy.dtype, device=dy.device) if out is None else out
        off = offsets.tolist()
        for g in range(G):
            s, e = off[g], off[g + 1]
            if e > s:
                y[s:e] = _lib_mm(dy[s:e], w[g]).to(y.dtype)
        return y
    assert N % 64 == 0, 'grouped dgrad needs the contraction (N) to be a multiple of 64'
    d2 = _row_major_2d(dy)
    w2 = w.contiguous().view(G * N, K)
    c = _out(out, (R, K), torch.bfloat16, dy.device, False)
    _launch(d2, N, R, d2.stride(0), False, w2, K, G * N, K, True, c, c.stride(0), 0, R, K, N, 1.0, None, False,
            mode=GROUPED_M, num_groups=G, offsets=offsets, b_group_rows=N)
    return c


def grouped_mm_tn(dy: torch.Tensor, x: torch.Tensor, offsets: torch.Tensor, out: Optional[torch.Tensor] = None,
                  out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    """``dw[g] = dy[rows g]^T @ x[rows g]`` -> ``[G, N, K]``; padded rows inside a group must be zero."""
    _check_offsets(offsets)
    G = offsets.numel() - 1
    N, K = dy.shape[-1], x.shape[-1]
    if not _use_cuda(dy, x, offsets):
        y = torch.zeros(G, N, K, dtype=torch.float32, device=dy.device)
        off = offsets.tolist()
        for g in range(G):
            s, e = off[g], off[g + 1]
            if e > s:
                y[g] = _lib_mm(dy[s:e].t(), x[s:e])
        if out is not None:
            if accumulate:
                out.add_(y.to(out.dtype))
            else:
                out.copy_(y.to(out.dtype))
            return out
        return y.to(out_dtype or dy.dtype)
    d2, x2 = _row_major_2d(dy), _row_major_2d(x)
    R = d2.shape[0]
    c = _out(out, (G, N, K), out_dtype or torch.bfloat16, dy.device, accumulate)
    assert c.is_contiguous()
    _launch(d2, N, R, d2.stride(0), True, x2, K, R, x2.stride(0), True, c, K, N * K, N, K, 0, 1.0, None, accumulate,
            mode=GROUPED_K, num_groups=G, offsets=offsets)
    return c
