"""Tensor-parallel linear as one autograd function: GEMMs on the tcgen05 engine, collectives either
fused into the GEMM kernel over peer memory (``parallel/fused_comm.py``, when set up) or through
``torch.distributed`` (baseline / CPU).

Modes
  ``None``      plain ``y = x W^T + b``
  ``'column'``  W is sharded on its output dim.  With sequence parallelism the input ``[T/tp, K]`` is
                all-gathered first (forward) and its gradient reduce-scattered (backward); without it the
                input gradient is all-reduced.
  ``'row'``     W is sharded on its input dim.  The partial outputs are reduce-scattered (sequence
                parallel) or all-reduced; backward all-gathers the output gradient.

Weight gradients go straight into ``weight.main_grad`` (fp32, accumulated by the GEMM epilogue) when
that attribute exists — the distributed optimizer owns those buffers — and ``weight.grad`` otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..parallel import mappings as M
from ..parallel import state as ps
from . import gemm


@dataclass(frozen=True)
class LinearSpec:
    mode: Optional[str] = None        # None | 'column' | 'row'
    sequence_parallel: bool = False
    group: str = 'tp'
    gather_output: bool = False       # column: all-gather the output on the last dim
    input_is_parallel: bool = True    # row: input already sharded on its last dim
    skip_weight_grad: bool = False
    allreduce_dgrad: bool = True      # column without SP: all-reduce dx (False when the caller does it later)
    fp8: bool = False                 # block-scaled fp8 forward and data-gradient GEMMs (weight gradient stays bf16)


def _weight_grad(weight: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor):
    """dW = dy^T x, fused into ``main_grad`` when the optimizer provides it."""
    mg = getattr(weight, 'main_grad', None)
    if mg is not None:
        gemm.mm_tn(dy2, x2, out=mg, accumulate=True)
        hook = getattr(weight, 'grad_ready_hook', None)
        if hook is not None:
            hook()
        return None
    return gemm.mm_tn(dy2, x2, out_dtype=weight.dtype)


def _fused():
    from ..parallel import fused_comm
    return fused_comm


def _use_fp8(spec: 'LinearSpec', x2: torch.Tensor, weight: torch.Tensor) -> bool:
    if not spec.fp8:
        return False
    from . import fp8
    return fp8.eligible(x2, weight)


def _mm_nt(x2, weight, bias, use_fp8: bool):
    if use_fp8:
        from . import fp8
        return fp8.mm_nt(x2, weight, bias)
    return gemm.mm_nt(x2, weight, bias=bias)


def _mm_nn(dy2, weight, use_fp8: bool):
    if use_fp8:
        from . import fp8
        return fp8.mm_nn(dy2, weight)
    return gemm.mm_nn(dy2, weight)


class _LinearFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, bias, spec: LinearSpec):
        ctx.spec = spec
        ctx.x_shape = x.shape
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        n = ps.get_world_size(spec.group) if spec.mode else 1
        ctx.n = n
        ctx.has_bias = bias is not None
        f8 = ctx.fp8 = _use_fp8(spec, x2, weight)
        if spec.mode == 'column' and spec.sequence_parallel and n > 1:
            fc = _fused()
            res = fc.all_gather_gemm(x2, weight, bias, spec.group) if (not f8 and fc.enabled(x2, weight, spec.group)) \
                else None
            if res is not None:
                y, x_full = res
            else:
                x_full = M.all_gather_dim0(x2, spec.group)
                y = _mm_nt(x_full, weight, bias, f8)
            # the gathered input feeds the weight gradient; under per-layer recompute it lives only briefly
            ctx.save_for_backward(x_full, weight)
            return y
        if spec.mode == 'row' and n > 1:
            if spec.sequence_parallel:
                fc = _fused()
                y = fc.gemm_reduce_scatter(x2, weight, spec.group) if (not f8 and fc.enabled(x2, weight, spec.group)) \
                    else None
                if y is None:
                    y = M.reduce_scatter_dim0(_mm_nt(x2, weight, None, f8), spec.group)
            else:
                y = M.all_reduce(_mm_nt(x2, weight, None, f8), spec.group)
            if bias is not None:
                y = y + bias
            ctx.save_for_backward(x2, weight)
            return y
        y = _mm_nt(x2, weight, bias, f8)
        ctx.save_for_backward(x2, weight)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        spec: LinearSpec = ctx.spec
        x2, weight = ctx.saved_tensors
        n = ctx.n
        N = weight.shape[0]
        dy2 = dy.reshape(-1, N)
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1] and not spec.skip_weight_grad
        dx = dw = db = None
        f8 = ctx.fp8
        if spec.mode == 'column' and spec.sequence_parallel and n > 1:
            x_full = x2  # saved gathered input
            if need_dx:
                fc = _fused()
                fused = not f8 and fc.enabled(dy2, weight, spec.group)
                dx = fc.gemm_reduce_scatter_nn(dy2, weight, spec.group) if fused else None
                if dx is None:
                    dx = M.reduce_scatter_dim0(_mm_nn(dy2, weight, f8), spec.group)
            if need_dw:
                dw = _weight_grad(weight, dy2, x_full)
            if ctx.has_bias:
                db = dy2.float().sum(0).to(dy.dtype)
            return dx, dw, db, None
        if spec.mode == 'row' and n > 1:
            if spec.sequence_parallel:
                fc = _fused()
                res = None
                if need_dx and not f8 and fc.enabled(dy2, weight, spec.group):
                    res = fc.all_gather_gemm_nn(dy2, weight, spec.group)
                if res is not None:
                    dx, dy_full = res
                else:
                    dy_full = M.all_gather_dim0(dy2, spec.group)
                    if need_dx:
                        dx = _mm_nn(dy_full, weight, f8)
            else:
                dy_full = dy2
                if need_dx:
                    dx = _mm_nn(dy_full, weight, f8)
            if need_dw:
                dw = _weight_grad(weight, dy_full, x2)
            if ctx.has_bias:
                db = dy2.float().sum(0).to(dy.dtype)
            return (dx.view(ctx.x_shape) if dx is not None else None), dw, db, None
        if need_dx:
            dx = _mm_nn(dy2, weight, f8)
            if spec.mode == 'column' and n > 1 and spec.allreduce_dgrad:
                dx = M.all_reduce(dx, spec.group)
            dx = dx.view(ctx.x_shape)
        if need_dw:
            dw = _weight_grad(weight, dy2, x2)
        if ctx.has_bias:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           spec: LinearSpec = LinearSpec()) -> torch.Tensor:
    if weight.dtype != x.dtype:
        x = x.to(weight.dtype)
    y = _LinearFn.apply(x, weight, bias, spec)
    if spec.mode == 'column' and spec.gather_output:
        y = M.gather_from_tensor_model_parallel_region(y, spec.group)
    return y
