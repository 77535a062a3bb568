"""Fused MoE token exchange on the in-tree kernels (``csrc/moe/moe_kernels.cu``).

Forward of one MoE layer on a rank:

1. router kernel -> probabilities, expert indices, per-expert counts, written straight into this rank's *published*
   region of a symmetric workspace together with a copy of the activations;
2. ``READY`` flag to all ranks of the expert-parallel group; wait for everybody's;
3. layout kernel (padded segment offsets from all ranks' counts), then the pull-dispatch kernel: the owner of an
   expert reads the routed rows out of the sources' published activations over NVLink into its expert-sorted GEMM
   input (ordinary local memory, so it can be kept for backward) and records where every copy went;
4. grouped expert GEMMs; the second one writes into the symmetric output buffer;
5. ``DONE`` flag; each source pulls and sums its ``k`` result rows (combine kernel).

Backward runs the same kernels with the saved row maps: gradient rows are pulled by the owners, expert backward
runs, input-gradient rows and the gradients of the routing probabilities are pulled back by the sources.

Workspaces are double buffered by call parity (see ``parallel/symm.py`` for the argument why that is sufficient).
With an expert-parallel size of one everything is local and no flags are exchanged.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import _lib
from ..parallel import state as ps
from ..parallel import symm

_int, _f, _u = ctypes.c_int, ctypes.c_float, ctypes.c_uint
FLAG_BYTES = 65536
F_READY, F_DONE = 0, 16
PAD = 128


def available(x: torch.Tensor) -> bool:
    if os.environ.get('MCB200_FUSED_MOE', '1') == '0':
        return False
    if not (x.is_cuda and x.dtype == torch.bfloat16 and _lib.available()):
        return False
    ep = ps.get_world_size('ep')
    return ep == 1 or (ep <= 8 and symm.is_supported())


def _arr(ptrs: List[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


@dataclass
class _Region:
    """Offsets of one parity half of a workspace."""
    x: int
    idx: int
    probs: int
    counts: int
    sent: int
    out: int
    scalar: int
    size: int


class ExchangeBuffers:
    """The exchange buffers of one direction as one layer call sees them: the shared allocation plus this call's token
    count ``T`` (calls of different sizes share an allocation laid out for the largest)."""

    def __init__(self, alloc: '_ExchangeAllocation', T: int):
        self._alloc = alloc
        self.T = T

    def __getattr__(self, name):
        return getattr(self._alloc, name)

    def sort_routing(self, parity: int):
        """Sorts the published routing of this rank by expert (``order`` / ``eoff`` regions) for the fused
        pull + GEMM kernel of the owners."""
        T, k, E = self.T, self.k, self.E
        rc = _lib.lib().mcb_moe_sort(_lib.ptr(self.view('idx', parity, (T * k,), torch.int32)),
                                     _lib.ptr(self.view('counts', parity, (E,), torch.int32)), _int(T * k), _int(E),
                                     _lib.ptr(self.view('eoff', parity, (E + 1,), torch.int32)),
                                     _lib.ptr(self.view('order', parity, (T * k,), torch.int32)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_moe_sort')


class _ExchangeAllocation:
    """Published/received buffers of one direction (forward or backward), laid out for up to ``T_alloc`` tokens."""

    def __init__(self, tag: str, T: int, H: int, k: int, E: int, capacity: int, device):
        self.tag, self.T_alloc, self.H, self.k, self.E, self.cap = tag, T, H, k, E, capacity
        self.world = ps.get_world_size('ep')
        self.rank = ps.get_rank_in('ep') if self.world > 1 else 0
        self.device = device

        def al(n):
            return (n + 1023) // 1024 * 1024

        o = 0
        offs = {}
        for name, nbytes in (('x', T * H * 2), ('idx', T * k * 4), ('probs', T * k * 4), ('counts', E * 4),
                             ('sent', T * k * 4), ('out', capacity * H * 2), ('scalar', capacity * 4),
                             ('order', T * k * 4), ('eoff', (E + 1) * 4),
                             # one slot per routing entry: the owners' last GEMM of a direction writes result rows
                             # (and per-entry scalars) straight into them
                             ('slots', T * k * H * 2), ('sslots', T * k * 4)):
            offs[name] = o
            o += al(nbytes)
        self.half = o
        self.offs = offs
        total = FLAG_BYTES + 2 * self.half
        if self.world > 1:
            self.ws_tag = f'moe_{tag}_{T}_{H}_{k}_{E}_{capacity}'
            self.ws = symm.get_workspace('ep', total, self.ws_tag)
            self.base_ptrs = self.ws.peer_ptrs
            self.buf = self.ws.buffer
        else:
            self.ws = None
            self.buf = torch.zeros(total, dtype=torch.uint8, device=device)
            self.base_ptrs = [self.buf.data_ptr()]
        self.epoch = 0
        self._ptr_cache: Dict[Tuple[str, int], ctypes.Array] = {}
        # "block landed" flags of the fused pull + GEMM kernel (local memory; they carry the epoch of the launch that
        # filled the block, so they are never cleared)
        # per block: the flag, then (second half) the counter of landed quarters
        self.blk_flags = torch.zeros(2 * max(1, capacity // PAD), dtype=torch.int32, device=device)
        self.pull_epoch = 0

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def next_pull_epoch(self) -> int:
        self.pull_epoch += 1
        return self.pull_epoch

    def off(self, name: str, parity: int) -> int:
        return FLAG_BYTES + parity * self.half + self.offs[name]

    def view(self, name: str, parity: int, shape, dtype) -> torch.Tensor:
        o = self.off(name, parity)
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.buf[o:o + nbytes].view(dtype).view(*shape)

    def ptrs(self, name: str, parity: int):
        key = (name, parity)
        a = self._ptr_cache.get(key)
        if a is None:
            a = _arr([p + self.off(name, parity) for p in self.base_ptrs])
            self._ptr_cache[key] = a
        return a

    def flag_ptrs(self):
        key = ('flags', 0)
        a = self._ptr_cache.get(key)
        if a is None:
            a = _arr(list(self.base_ptrs))
            self._ptr_cache[key] = a
        return a

    def signal(self, base: int, value: int):
        if self.world == 1:
            return
        _lib.check_rc(_lib.lib().mcb_flag_signal(self.flag_ptrs(), _int(self.world), _int(self.rank), _int(base),
                                                 _u(value), _lib.stream_ptr()), 'mcb_flag_signal')

    def wait(self, base: int, value: int):
        if self.world == 1:
            return
        _lib.check_rc(_lib.lib().mcb_flag_wait(self.flag_ptrs(), _int(self.world), _int(self.rank), _int(base),
                                               _u(value), _lib.ptr(_lib.status_word(self.device)),
                                               _lib.stream_ptr()), 'mcb_flag_wait')


_BUFFERS: Dict[Tuple, _ExchangeAllocation] = {}


def _buffers(tag, T, H, k, E, cap, device) -> ExchangeBuffers:
    """One set of exchange buffers per (direction, layer shape), laid out for the largest token count and capacity
    seen so far: a larger micro-batch re-allocates (a collective call: every rank of the group sees the same sizes),
    smaller ones reuse the regions, so variable-length micro-batches do not pile up peer-mapped workspaces.  Calls
    still in flight (saved for a later backward) keep the buffers they started with."""
    # the expert-parallel group is part of the identity: an allocation holds that group's peer mappings
    key = (tag, H, k, E, device.index, tuple(ps.get_group_ranks('ep')))
    a = _BUFFERS.get(key)
    if a is None or T > a.T_alloc or cap > a.cap:
        t_new, cap_new = T, cap
        if a is not None:
            t_new, cap_new = max(T, a.T_alloc), max(cap, a.cap)
            if a.ws is not None:
                symm.release_workspace('ep', a.ws_tag)
        a = _ExchangeAllocation(tag, t_new, H, k, E, cap_new, device)
        _BUFFERS[key] = a
    return ExchangeBuffers(a, T)


_GROWN_FACTOR: Optional[float] = None     # raised by ``grow_capacity`` after an overflow; never shrinks


def grow_capacity() -> float:
    """Doubles the capacity factor used for every later call (the trainer calls this on all ranks after a step in
    which a rank received more rows than its buffer holds, then repeats the step)."""
    global _GROWN_FACTOR
    base = _GROWN_FACTOR or float(os.environ.get('MCB200_MOE_CAPACITY_FACTOR', 2.0))
    _GROWN_FACTOR = base * 2.0
    return _GROWN_FACTOR


def capacity_rows(T: int, k: int, El: int, world: int, factor: Optional[float]) -> int:
    """Rows of the receive buffer: ``factor`` x the balanced load plus worst-case padding, capped by the true worst
    case (every copy of every rank lands here).

    The model config's ``moe_expert_capacity_factor`` is normally unset (dropless).  No token is ever dropped here
    either: the buffer starts at twice the balanced load, and a routing that does not fit raises the overflow
    status, which suppresses the optimizer update on the device; the trainer then grows the factor and repeats the
    step (``Trainer.train_step``).  The true worst case is ``world`` x the balanced load, which at 8 ranks would
    quadruple the activation memory of every MoE layer for a case that near-uniform routing never meets."""
    f = float(os.environ.get('MCB200_MOE_CAPACITY_FACTOR', factor or 2.0))
    if _GROWN_FACTOR is not None:
        f = max(f, _GROWN_FACTOR)
    worst = world * T * k
    rows = min(worst, int(f * T * k)) + El * PAD
    return (rows + PAD - 1) // PAD * PAD


# ---------------------------------------------------------------------------------------------------------------
class _RouterFn(torch.autograd.Function):
    """logits -> (probs [T,k], idx [T,k] int32, score_sum [E]); counts [E] int32 are written into ``counts_out``."""

    @staticmethod
    def forward(ctx, logits, bias, valid, k, sigmoid, renorm, groups, group_topk, scaling, probs_out, idx_out,
                counts_out):
        T, E = logits.shape
        logits = logits.contiguous()
        scores = torch.empty((T, E), dtype=torch.float32, device=logits.device)
        score_sum = torch.zeros(E, dtype=torch.float32, device=logits.device)
        counts_out.zero_()
        rc = _lib.lib().mcb_router_fwd(_lib.ptr(logits), _lib.ptr(bias), _lib.ptr(valid), _lib.ptr(probs_out),
                                       _lib.ptr(idx_out), _lib.ptr(scores), _lib.ptr(counts_out), _lib.ptr(score_sum),
                                       _int(T), _int(E), _int(k), _int(int(sigmoid)), _int(int(renorm)),
                                       _int(groups or 0), _int(group_topk or 0), _f(scaling), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_router_fwd')
        idx_saved = idx_out.clone()
        ctx.save_for_backward(scores, idx_saved, valid)
        ctx.meta = (k, sigmoid, renorm, scaling)
        ctx.mark_non_differentiable(idx_saved)
        return probs_out.clone(), idx_saved, score_sum

    @staticmethod
    def backward(ctx, dprobs, _didx, dscore_sum):
        scores, idx, valid = ctx.saved_tensors
        k, sigmoid, renorm, scaling = ctx.meta
        T, E = scores.shape
        dlogits = torch.empty_like(scores)
        dprobs = dprobs.float().contiguous() if dprobs is not None else torch.zeros((T, k), device=scores.device)
        dvec = dscore_sum.float().contiguous() if dscore_sum is not None else None
        rc = _lib.lib().mcb_router_bwd(_lib.ptr(dprobs), _lib.ptr(idx), _lib.ptr(scores), _lib.ptr(dvec),
                                       _lib.ptr(valid), _lib.ptr(dlogits), _int(T), _int(E), _int(k),
                                       _int(int(sigmoid)), _int(int(renorm)), _f(scaling), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_router_bwd')
        return (dlogits,) + (None,) * 11


def router_supported(E: int, k: int, groups: Optional[int]) -> bool:
    if E % 32 or E > 512 or k > 16:
        return False
    if groups and groups > 1:
        epl = E // 32
        if E % groups or (E // groups) % epl:
            return False
        lpg = (E // groups) // epl
        if lpg < 1 or lpg & (lpg - 1):
            return False
    return True


@dataclass
class DispatchState:
    fwd: ExchangeBuffers
    bwd: ExchangeBuffers
    parity: int
    seg_off: torch.Tensor      # [El+1] int32 (the grouped GEMM offsets)
    row_src: torch.Tensor      # [cap] int32
    sent_row: Optional[torch.Tensor] = None   # [T,k] int32, saved copy
    idx: Optional[torch.Tensor] = None


class _DispatchFn(torch.autograd.Function):
    """(x [T,H], probs [T,k]) -> (xp [cap,H], row_probs [cap]) on the expert owners."""

    @staticmethod
    def forward(ctx, x, probs, idx, st: DispatchState, El: int):
        b = st.fwd
        T, H, k, E = b.T, b.H, b.k, b.E
        par = st.parity
        epoch = b.epoch
        b.view('x', par, (T, H), torch.bfloat16).copy_(x)
        b.view('probs', par, (T, k), torch.float32).copy_(probs.float())
        # idx and counts were written into the published region by the router kernel
        b.signal(F_READY, epoch)
        b.wait(F_READY, epoch)
        dev = x.device
        src_off = torch.empty(b.world * El, dtype=torch.int32, device=dev)
        rc = _lib.lib().mcb_moe_layout(b.ptrs('counts', par), _int(b.world), _int(b.rank), _int(E), _int(El),
                                       _lib.ptr(st.seg_off), _lib.ptr(src_off), _int(b.cap),
                                       _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_moe_layout')
        xp = torch.zeros((b.cap, H), dtype=torch.bfloat16, device=dev)
        row_probs = torch.zeros(b.cap, dtype=torch.float32, device=dev)
        st.row_src.fill_(-1)
        cursor = torch.zeros(b.world * El, dtype=torch.int32, device=dev)
        rc = _lib.lib().mcb_moe_pull_dispatch(b.ptrs('x', par), b.ptrs('idx', par), b.ptrs('probs', par),
                                              b.ptrs('sent', par), _int(b.world), _int(b.rank), _int(T), _int(k),
                                              _int(E), _int(El), _int(H), _int(b.cap), _lib.ptr(st.seg_off),
                                              _lib.ptr(src_off), _lib.ptr(cursor), _lib.ptr(xp), _lib.ptr(row_probs),
                                              _lib.ptr(st.row_src), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_moe_pull_dispatch')
        ctx.st = st
        ctx.meta = (T, H, k, E, El)
        ctx.pdtype = probs.dtype
        return xp, row_probs

    @staticmethod
    def backward(ctx, dxp, drow_probs):
        st: DispatchState = ctx.st
        T, H, k, E, El = ctx.meta
        b = st.bwd
        par = b.epoch & 1   # same call whose first half ran in _CombineFn.backward
        epoch = b.epoch
        # owners publish their input-gradient rows and probability gradients, sources pull them back
        b.view('out', par, (b.cap, H), torch.bfloat16).copy_(dxp)
        sc = b.view('scalar', par, (b.cap,), torch.float32)
        if drow_probs is not None:
            sc.copy_(drow_probs.float())
        else:
            sc.zero_()
        b.signal(F_DONE, epoch)
        b.wait(F_DONE, epoch)
        dx = torch.empty((T, H), dtype=torch.bfloat16, device=dxp.device)
        dprobs = torch.empty((T, k), dtype=torch.float32, device=dxp.device)
        rc = _lib.lib().mcb_moe_combine(b.ptrs('out', par), b.ptrs('scalar', par), _int(b.world), _int(T), _int(k),
                                        _int(El), _int(H), _lib.ptr(st.idx), _lib.ptr(st.sent_row), _lib.ptr(dx),
                                        _lib.ptr(dprobs), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_moe_combine')
        return dx, dprobs.to(ctx.pdtype), None, None, None


class _CombineFn(torch.autograd.Function):
    """y rows on the owners (already in the symmetric output buffer) -> out [T,H] on the sources."""

    @staticmethod
    def forward(ctx, y, st: DispatchState, El: int):
        b = st.fwd
        T, H, k = b.T, b.H, b.k
        par = st.parity
        epoch = b.epoch
        out_buf = b.view('out', par, (b.cap, H), torch.bfloat16)
        if y.data_ptr() != out_buf.data_ptr():
            out_buf.copy_(y)
        b.signal(F_DONE, epoch)
        b.wait(F_DONE, epoch)
        idx = b.view('idx', par, (T, k), torch.int32)
        sent = b.view('sent', par, (T, k), torch.int32)
        out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
        rc = _lib.lib().mcb_moe_combine(b.ptrs('out', par), None, _int(b.world), _int(T), _int(k), _int(El), _int(H),
                                        _lib.ptr(idx), _lib.ptr(sent), _lib.ptr(out), None, _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_moe_combine')
        st.sent_row = sent.clone()   # the published tables are reused two calls later
        st.idx = idx.clone()
        ctx.st = st
        ctx.meta = (T, H, k, El)
        return out

    @staticmethod
    def backward(ctx, dout):
        st: DispatchState = ctx.st
        T, H, k, El = ctx.meta
        b = st.bwd
        epoch = b.next_epoch()
        par = epoch & 1
        b.view('x', par, (T, H), torch.bfloat16).copy_(dout)
        b.signal(F_READY, epoch)
        b.wait(F_READY, epoch)
        dy = torch.empty((b.cap, H), dtype=torch.bfloat16, device=dout.device)
        rc = _lib.lib().mcb_moe_pull_rows(b.ptrs('x', par), _int(b.world), _int(T), _int(k), _int(H),
                                          _lib.ptr(st.row_src), _int(b.cap), _lib.ptr(dy), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_moe_pull_rows')
        return dy, None, None


def _weight_grad_grouped(weight, dy, x, offsets):
    """dW of a stacked expert weight: straight into ``main_grad`` when the optimizer provides it."""
    from ..ops import gemm
    mg = getattr(weight, 'main_grad', None)
    if mg is not None:
        gemm.grouped_mm_tn(dy, x, offsets, out=mg, accumulate=True)
        hook = getattr(weight, 'grad_ready_hook', None)
        if hook is not None:
            hook()
        return None
    return gemm.grouped_mm_tn(dy, x, offsets, out_dtype=weight.dtype)


def _pull_gemm(b: ExchangeBuffers, par: int, mode: int, st: 'DispatchState', El: int, rows_region: str, weight,
               b_mn: bool, xp, row_probs, out):
    """Launches the fused pull + grouped GEMM kernel on ``b``'s published regions of parity ``par``."""
    T, H, k, E = b.T, b.H, b.k, b.E
    G, d1, d2 = weight.shape
    w2 = weight.view(G * d1, d2)
    if b_mn:            # weight [El, H(contraction), N]: rows of the 2-D view are contraction indices
        N, b_inner, b_outer, group_rows = d2, d2, G * d1, d1
    else:               # weight [El, N, H]
        N, b_inner, b_outer, group_rows = d1, d2, G * d1, d1
    fwd = mode == 0
    rc = _lib.lib().mcb_moe_pull_gemm(
        b.ptrs(rows_region, par), b.ptrs('order', par) if fwd else None, b.ptrs('eoff', par) if fwd else None,
        b.ptrs('probs', par) if fwd else None, b.ptrs('sent', par) if fwd else None, _int(b.world), _int(b.rank),
        _int(T), _int(k), _int(E), _int(El), _int(H), _int(N), _int(b.cap), _int(mode), _lib.ptr(st.seg_off),
        _lib.ptr(st.row_src), _lib.ptr(row_probs), _lib.ptr(xp), _lib.ptr(b.blk_flags), _u(b.next_pull_epoch()),
        _lib.ptr(w2), ctypes.c_longlong(b_inner), ctypes.c_longlong(b_outer), ctypes.c_longlong(w2.stride(0)),
        _int(int(b_mn)), _int(group_rows), _lib.ptr(out), ctypes.c_longlong(out.stride(0)),
        _lib.ptr(_lib.status_word(xp.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_moe_pull_gemm')




def _gemm_scatter(b: ExchangeBuffers, par: int, st: 'DispatchState', El: int, a2: torch.Tensor, weight: torch.Tensor,
                  b_mn: bool, scalar: Optional[torch.Tensor]):
    """Grouped expert GEMM over the expert-sorted rows ``a2 [cap, K]`` whose epilogue sends every result row to the
    slot of the routing entry it belongs to on the entry's source rank (``slots`` region, over NVLink for remote
    sources); ``scalar [cap]`` (fp32, optional) travels the same way into ``sslots``."""
    G, d1, d2 = weight.shape
    w2 = weight.view(G * d1, d2)
    if b_mn:            # weight [El, K(contraction), N]
        K, N, b_inner, b_outer, group_rows = d1, d2, d2, G * d1, d1
    else:               # weight [El, N, K]
        K, N, b_inner, b_outer, group_rows = d2, d1, d2, G * d1, d1
    assert a2.shape == (b.cap, K) and a2.is_contiguous() and N == b.H
    rc = _lib.lib().mcb_moe_gemm_scatter(
        _lib.ptr(a2), _lib.ptr(w2), ctypes.c_longlong(b_inner), ctypes.c_longlong(b_outer),
        ctypes.c_longlong(w2.stride(0)), _int(int(b_mn)), _int(group_rows), b.ptrs('slots', par),
        b.ptrs('sslots', par) if scalar is not None else None, _lib.ptr(scalar), _lib.ptr(st.seg_off),
        _lib.ptr(st.row_src), _int(b.world), _int(b.T), _int(b.k), _int(El), _int(K), _int(N), _int(b.cap),
        _lib.ptr(_lib.status_word(a2.device)), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_moe_gemm_scatter')


def scatter_enabled() -> bool:
    """The last GEMM of each direction pushes its rows to the sources' slots (``MCB200_MOE_SCATTER=0``: it writes the
    owner's buffer and the sources pull and sum with ``moe_combine``)."""
    return os.environ.get('MCB200_MOE_SCATTER', '0') != '0'


def _sum_slots(b: ExchangeBuffers, par: int, sent: torch.Tensor) -> torch.Tensor:
    """Per token, the fixed-order sum of the ``k`` result rows the owners wrote into this rank's slots."""
    out = torch.empty((b.T, b.H), dtype=torch.bfloat16, device=sent.device)
    rc = _lib.lib().mcb_moe_sum_slots(_lib.ptr(b.view('slots', par, (b.T * b.k, b.H), torch.bfloat16)), _lib.ptr(sent),
                                      _int(b.T), _int(b.k), _int(b.H), _lib.ptr(out), _lib.stream_ptr())
    _lib.check_rc(rc, 'mcb_moe_sum_slots')
    return out


def pull_gemm_supported(experts, config, El: int, H: int) -> bool:
    """The fused dispatch + expert GEMM applies to plain stacked bf16 expert weights without biases, probabilities
    applied after the first layer and at most 64 local experts."""
    from .moe import GroupedLinear, GroupedMLP
    if os.environ.get('MCB200_MOE_FUSED_GEMM', '1') == '0':
        return False
    if type(experts) is not GroupedMLP or config.moe_apply_probs_on_input:
        return False
    for lin in (experts.linear_fc1, experts.linear_fc2):
        if type(lin) is not GroupedLinear or lin.bias is not None or lin.weight.dtype != torch.bfloat16:
            return False
    f = experts.linear_fc2.weight.shape[2]
    return El <= 64 and H % 64 == 0 and f % 64 == 0 and experts.linear_fc1.weight.shape[1] % 8 == 0


class _DispatchFc1Fn(torch.autograd.Function):
    """(x [T,H], probs [T,k], w1 [El,N,H]) -> (h [cap,N], row_probs [cap]): the owners pull their routed rows and
    run the first expert layer in one launch; the exchange hides behind the GEMM block by block."""

    @staticmethod
    def forward(ctx, x, probs, idx, w1, st: 'DispatchState', El: int):
        b = st.fwd
        T, H, k = b.T, b.H, b.k
        par, epoch = st.parity, b.epoch
        b.view('x', par, (T, H), torch.bfloat16).copy_(x)
        b.view('probs', par, (T, k), torch.float32).copy_(probs.float())
        b.sort_routing(par)                   # idx and counts were published by the router
        b.signal(F_READY, epoch)
        b.wait(F_READY, epoch)
        dev = x.device
        xp = torch.empty((b.cap, H), dtype=torch.bfloat16, device=dev)
        h = torch.empty((b.cap, w1.shape[1]), dtype=torch.bfloat16, device=dev)
        row_probs = torch.empty(b.cap, dtype=torch.float32, device=dev)
        _pull_gemm(b, par, 0, st, El, 'x', w1, False, xp, row_probs, h)
        ctx.save_for_backward(xp, w1)
        ctx.st, ctx.El, ctx.pdtype = st, El, probs.dtype
        return h, row_probs

    @staticmethod
    def backward(ctx, dh, drow_probs):
        from ..ops import gemm
        xp, w1 = ctx.saved_tensors
        st, El = ctx.st, ctx.El
        b = st.bwd
        T, H, k = b.T, b.H, b.k
        dh = dh.contiguous()
        par, epoch = b.epoch & 1, b.epoch     # same call whose first half ran in _Fc2CombineFn.backward
        # the data-gradient GEMM of the first layer sends every input-gradient row (and the gradient of its routing
        # probability) straight to the slot of its entry on the source rank; the sources then add their k slots
        if scatter_enabled():
            sc = drow_probs.float().contiguous() if drow_probs is not None else None
            _gemm_scatter(b, par, st, El, dh, w1, True, sc)
            dw1 = _weight_grad_grouped(w1, dh, xp, st.seg_off) if ctx.needs_input_grad[3] else None
            b.signal(F_DONE, epoch)
            b.wait(F_DONE, epoch)
            dx = _sum_slots(b, par, st.sent_row)
            if sc is not None:
                dprobs = torch.where(st.sent_row >= 0, b.view('sslots', par, (T, k), torch.float32), 0.0)
            else:
                dprobs = torch.zeros((T, k), dtype=torch.float32, device=dh.device)
            return dx, dprobs.to(ctx.pdtype), None, dw1, None, None
        # owners publish their input-gradient rows (written by the GEMM straight into the symmetric region) and the
        # probability gradients, sources pull them back
        gemm.grouped_mm_nn(dh, w1, st.seg_off, out=b.view('out', par, (b.cap, H), torch.bfloat16))
        dw1 = _weight_grad_grouped(w1, dh, xp, st.seg_off) if ctx.needs_input_grad[3] else None
        sc = b.view('scalar', par, (b.cap,), torch.float32)
        if drow_probs is not None:
            sc.copy_(drow_probs.float())
        else:
            sc.zero_()
        b.signal(F_DONE, epoch)
        b.wait(F_DONE, epoch)
        dx = torch.empty((T, H), dtype=torch.bfloat16, device=dh.device)
        dprobs = torch.empty((T, k), dtype=torch.float32, device=dh.device)
        rc = _lib.lib().mcb_moe_combine(b.ptrs('out', par), b.ptrs('scalar', par), _int(b.world), _int(T), _int(k),
                                        _int(El), _int(H), _lib.ptr(st.idx), _lib.ptr(st.sent_row), _lib.ptr(dx),
                                        _lib.ptr(dprobs), _lib.stream_ptr())
        _lib.check_rc(rc, 'mcb_moe_combine')
        return dx, dprobs.to(ctx.pdtype), None, dw1, None, None


class _Fc2CombineFn(torch.autograd.Function):
    """(a [cap,F], w2 [El,H,F]) -> out [T,H]: the second expert layer's epilogue sends every result row to its entry's
    slot on the source rank, then the sources add their k slots.  Backward: the owners pull the output-gradient rows and
    run the data-gradient GEMM of the second layer in one launch."""

    @staticmethod
    def forward(ctx, a, w2, st: 'DispatchState', El: int):
        from ..ops import gemm
        b = st.fwd
        T, H, k = b.T, b.H, b.k
        par, epoch = st.parity, b.epoch
        scatter = scatter_enabled()
        if scatter:
            _gemm_scatter(b, par, st, El, a.contiguous(), w2, False, None)
        else:
            gemm.grouped_mm_nt(a, w2, st.seg_off, out=b.view('out', par, (b.cap, H), torch.bfloat16))
        b.signal(F_DONE, epoch)
        b.wait(F_DONE, epoch)
        idx = b.view('idx', par, (T, k), torch.int32)
        sent = b.view('sent', par, (T, k), torch.int32)
        if scatter:
            out = _sum_slots(b, par, sent)
        else:
            out = torch.empty((T, H), dtype=torch.bfloat16, device=a.device)
            rc = _lib.lib().mcb_moe_combine(b.ptrs('out', par), None, _int(b.world), _int(T), _int(k), _int(El),
                                            _int(H), _lib.ptr(idx), _lib.ptr(sent), _lib.ptr(out), None,
                                            _lib.stream_ptr())
            _lib.check_rc(rc, 'mcb_moe_combine')
        st.sent_row = sent.clone()   # the published tables are reused two calls later
        st.idx = idx.clone()
        ctx.save_for_backward(a, w2)
        ctx.st, ctx.El = st, El
        return out

    @staticmethod
    def backward(ctx, dout):
        a, w2 = ctx.saved_tensors
        st, El = ctx.st, ctx.El
        b = st.bwd
        T, H = b.T, b.H
        epoch = b.next_epoch()
        par = epoch & 1
        b.view('x', par, (T, H), torch.bfloat16).copy_(dout)
        b.signal(F_READY, epoch)
        b.wait(F_READY, epoch)
        dy = torch.empty((b.cap, H), dtype=torch.bfloat16, device=dout.device)
        da = torch.empty_like(a)
        _pull_gemm(b, par, 1, st, El, 'x', w2, True, dy, None, da)
        dw2 = _weight_grad_grouped(w2, dy, a, st.seg_off) if ctx.needs_input_grad[1] else None
        return da, dw2, None, None


class FusedMoEDispatcher:
    """Per-layer helper owned by ``MoELayer``; holds no parameters."""

    def __init__(self, config, num_local_experts: int):
        self.config = config
        self.El = num_local_experts
        self.E = config.num_moe_experts
        self.k = config.moe_router_topk

    def begin(self, T: int, H: int, device) -> DispatchState:
        world = ps.get_world_size('ep')
        cap = capacity_rows(T, self.k, self.El, world, self.config.moe_expert_capacity_factor)
        fwd = _buffers('f', T, H, self.k, self.E, cap, device)
        bwd = _buffers('b', T, H, self.k, self.E, cap, device)
        epoch = fwd.next_epoch()
        return DispatchState(fwd=fwd, bwd=bwd, parity=epoch & 1,
                             seg_off=torch.empty(self.El + 1, dtype=torch.int32, device=device),
                             row_src=torch.empty(fwd.cap, dtype=torch.int32, device=device))

    def route(self, st: DispatchState, logits: torch.Tensor, bias, valid, sigmoid, renorm, groups, group_topk, scaling):
        b = st.fwd
        probs_out = torch.empty((b.T, b.k), dtype=torch.float32, device=logits.device)
        idx_out = b.view('idx', st.parity, (b.T, b.k), torch.int32)
        counts_out = b.view('counts', st.parity, (b.E,), torch.int32)
        if valid is None:
            probs, idx, score_sum = _RouterFn.apply(logits, bias, None, b.k, sigmoid, renorm, groups, group_topk,
                                                    float(scaling or 1.0), probs_out, idx_out, counts_out)
            return probs, idx, score_sum, counts_out
        # Padded tokens are routed like any other token but do not enter the load statistics: the kernel's counts
        # (valid tokens only) go to the caller, the published counts, which size the exchange, cover every entry.
        stat_counts = torch.empty(b.E, dtype=torch.int32, device=logits.device)
        probs, idx, score_sum = _RouterFn.apply(logits, bias, valid.to(torch.uint8).contiguous(), b.k, sigmoid, renorm,
                                                groups, group_topk, float(scaling or 1.0), probs_out, idx_out,
                                                stat_counts)
        counts_out.copy_(torch.bincount(idx_out.reshape(-1).long(), minlength=b.E).to(torch.int32))
        return probs, idx, score_sum, stat_counts

    def publish_routing(self, st: DispatchState, idx: torch.Tensor):
        """Routing decided elsewhere (torch router): publish indices and per-expert counts for the exchange."""
        b = st.fwd
        b.view('idx', st.parity, (b.T, b.k), torch.int32).copy_(idx.to(torch.int32))
        counts = torch.bincount(idx.reshape(-1), minlength=b.E).to(torch.int32)
        b.view('counts', st.parity, (b.E,), torch.int32).copy_(counts)
        return counts

    def dispatch(self, st: DispatchState, x, probs, idx):
        return _DispatchFn.apply(x, probs, idx, st, self.El)

    def experts_fused(self, st: DispatchState, x, probs, idx, experts):
        """Dispatch + both expert layers + combine with the exchange fused into the expert GEMMs
        (``pull_gemm_supported`` decides whether this path applies)."""
        from ..ops.activation import glu
        cfg = self.config
        h, row_probs = _DispatchFc1Fn.apply(x, probs, idx, experts.linear_fc1.weight, st, self.El)
        if cfg.gated_linear_unit:
            a = glu(h, experts.kind, row_probs, cfg.activation_func_clamp_value or 0.0, cfg.glu_linear_offset)
        else:
            a = cfg.activation_func(h) * row_probs[:, None].to(h.dtype)
        return _Fc2CombineFn.apply(a, experts.linear_fc2.weight, st, self.El)

    def out_buffer(self, st: DispatchState) -> torch.Tensor:
        """Where the last expert GEMM should write so that the combine needs no copy."""
        b = st.fwd
        return b.view('out', st.parity, (b.cap, b.H), torch.bfloat16)

    def combine(self, st: DispatchState, y):
        return _CombineFn.apply(y, st, self.El)
