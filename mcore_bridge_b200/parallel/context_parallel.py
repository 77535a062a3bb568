"""Context-parallel attention.

Every CP rank holds, for each packed sequence, the zig-zag chunks ``r`` and ``2cp-1-r`` (``split_cp_inputs``), which
balances causal work.  Attention of the local queries needs all keys / values that precede them in their sequence.

On a GPU (head sizes the in-tree kernel covers) one autograd function does the whole exchange with in-tree kernels:

* forward: every rank writes its K / V into a symmetric buffer and the peer-memory all-gather kernel
  (``csrc/comm/dp_collectives.cu``) pulls the other ranks' slices over NVLink; the gathered rows are put into the order
  of the original token stream, where the keys a query may see form one contiguous range, and the attention kernel
  (``csrc/attention``, per-query key ranges) runs once over local queries x all keys;
* backward: the same kernel family gives dQ and the dK / dV of *all* keys; those go back into rank-major order and
  the peer-memory reduce-scatter kernel returns to every rank the fp32 sum of the gradients of its own keys.

The layout tensors (``CpLayout``) are computed on the device from ``cu_seqlens`` once per micro-batch and shared by all
layers; nothing synchronises with the host.  The reference reaches the same result through TransformerEngine
(``cp_comm_type``, ``src/mcore_bridge/config/model_config.py:240``, zig-zag split
``src/mcore_bridge/utils/megatron_utils.py:48-68``).

Elsewhere (CPU / gloo, head sizes or mask options the kernel lacks) K / V are all-gathered with ``torch.distributed``
(differentiable) and the masked-softmax reference or the generic attention op computes the same thing.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import state as ps


class _AllGatherTokens(torch.autograd.Function):
    """``[T_local, ...]`` -> ``[cp * T_local, ...]`` rank-major; backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, group_name):
        ctx.group_name = group_name
        n = ps.get_world_size(group_name)
        out = torch.empty((n * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=ps.get_group(group_name))
        return out

    @staticmethod
    def backward(ctx, g):
        n = ps.get_world_size(ctx.group_name)
        g = g.contiguous()
        if g.is_cuda:
            out = torch.empty((g.shape[0] // n, *g.shape[1:]), dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, group=ps.get_group(ctx.group_name))
            return out, None
        tmp = g.clone()
        dist.all_reduce(tmp, group=ps.get_group(ctx.group_name))
        r = ps.get_rank_in(ctx.group_name)
        c = g.shape[0] // n
        return tmp[r * c:(r + 1) * c].contiguous(), None


@dataclass
class CpLayout:
    """Index tensors of one micro-batch under context parallelism (all on the device of the activations).

    "Stream order" is the order of the original token stream; "rank-major" is ``[rank 0's tokens | rank 1's | ...]``,
    what an all-gather produces."""
    cp: int
    rank: int
    t_local: int
    gather_index: torch.Tensor      # int64 [T]: rank-major index of the token at each stream position
    scatter_index: torch.Tensor     # int64 [T]: stream position of the token at each rank-major index
    q_stream: torch.Tensor          # int64 [T_local]: stream position of each local token
    q_rel: torch.Tensor             # int64 [T_local]: position of each local token inside its sequence
    k_lo: torch.Tensor              # int32 [T_local]: first key (stream order) each local query sees
    k_hi: torch.Tensor              # int32 [T_local]: last key it sees (itself)
    q_lo: torch.Tensor              # int32 [T]: first local query that can see the key at each stream position
    q_hi: torch.Tensor              # int32 [T]: last one (empty range where none can)
    cu_local: torch.Tensor          # int32 [B+1]: sequence boundaries among the local tokens
    cu_full: torch.Tensor           # int32 [B+1]
    ring_lo: torch.Tensor           # int32 [cp, T_local]: first key, in rank j's local order, local query i sees
    ring_hi: torch.Tensor           # int32 [cp, T_local]: last one (lo > hi: none)
    ring_qlo: torch.Tensor          # int32 [cp, T_local]: first local query that can see token t of rank j
    ring_qhi: torch.Tensor          # int32 [cp, T_local]: last one (they bound the loops of the dK/dV kernel)


def compute_layout(cu_seqlens: Optional[torch.Tensor], t_local: int, cp: int, rank: int, device) -> CpLayout:
    """Vectorised on the device: no ``.tolist()``, no host synchronisation.  Every sequence length must be a multiple
    of ``2 * cp`` (what ``split_cp_inputs`` requires)."""
    T = t_local * cp
    if cu_seqlens is None:
        cu = torch.tensor([0, T], dtype=torch.int64, device=device)
    else:
        cu = cu_seqlens.to(device=device, dtype=torch.int64)
    B = cu.numel() - 1
    g = torch.arange(T, device=device)
    seg = torch.searchsorted(cu[1:].contiguous(), g, right=True).clamp(max=B - 1)
    S = cu[seg]
    n = cu[seg + 1] - S
    h = (n // (2 * cp)).clamp(min=1)
    rel = g - S
    c = torch.div(rel, h, rounding_mode='floor').clamp(max=2 * cp - 1)
    second = c >= cp
    rk = torch.where(second, 2 * cp - 1 - c, c)
    L0 = torch.div(S, cp, rounding_mode='floor')
    off = L0 + torch.where(second, h, torch.zeros_like(h)) + (rel - c * h)
    gather_index = rk * t_local + off
    scatter_index = torch.empty_like(gather_index)
    scatter_index[gather_index] = g
    q_stream = scatter_index[rank * t_local:(rank + 1) * t_local].contiguous()
    k_lo = S[q_stream].to(torch.int32)
    k_hi = q_stream.to(torch.int32)
    # local queries of a sequence sit at in-sequence positions [r h, (r+1) h) and [(2cp-1-r) h, (2cp-r) h), in that
    # order; the key at in-sequence position `rel` is seen by those with position >= rel
    before = (rel - rank * h).clamp(min=0).minimum(h) + (rel - (2 * cp - 1 - rank) * h).clamp(min=0).minimum(h)
    q_lo = L0 + before
    q_hi = L0 + 2 * h - 1
    none = before >= 2 * h
    q_lo = torch.where(none, torch.ones_like(q_lo), q_lo).to(torch.int32)
    q_hi = torch.where(none, torch.zeros_like(q_hi), q_hi).to(torch.int32)
    cu_local = torch.div(cu, cp, rounding_mode='floor').to(torch.int32)
    # Ring steps: rank j holds, per sequence, the chunks j and 2cp-1-j back to back (h tokens each, starting at local
    # index L0).  A query at in-sequence position rho sees a prefix of chunk j, and, only once chunk j is wholly
    # visible, a prefix of chunk 2cp-1-j: one contiguous range of rank j's local tokens.
    q_rel = q_stream - S[q_stream]
    hq, lq = h[q_stream], L0[q_stream]
    j = torch.arange(cp, device=device)[:, None]
    n1 = (q_rel[None, :] - j * hq[None, :] + 1).clamp(min=0).minimum(hq[None, :])
    n2 = (q_rel[None, :] - (2 * cp - 1 - j) * hq[None, :] + 1).clamp(min=0).minimum(hq[None, :])
    cnt = n1 + n2
    ring_lo = torch.where(cnt > 0, lq[None, :].expand(cp, -1), torch.ones_like(cnt)).to(torch.int32).contiguous()
    ring_hi = torch.where(cnt > 0, lq[None, :] + cnt - 1, torch.zeros_like(cnt)).to(torch.int32).contiguous()
    # q_lo / q_hi are indexed by stream position; rank j's token t sits at stream position scatter_index[j * tl + t]
    ring_qlo = q_lo[scatter_index].view(cp, t_local).contiguous()
    ring_qhi = q_hi[scatter_index].view(cp, t_local).contiguous()
    return CpLayout(cp, rank, t_local, gather_index, scatter_index, q_stream, q_rel, k_lo, k_hi, q_lo, q_hi, cu_local,
                    cu.to(torch.int32), ring_lo, ring_hi, ring_qlo, ring_qhi)


def get_layout(ctx, t_local: int, device) -> CpLayout:
    """The micro-batch's layout, computed on first use and kept in the forward context for the other layers."""
    lay = ctx.extra.get('cp_layout') if hasattr(ctx, 'extra') else None
    if lay is None or lay.t_local != t_local or lay.gather_index.device != torch.device(device):
        lay = compute_layout(ctx.cu_seqlens, t_local, ps.get_world_size('cp'), ps.get_rank_in('cp'), device)
        if hasattr(ctx, 'extra'):
            ctx.extra['cp_layout'] = lay
    return lay


# ---------------------------------------------------------------------------------------------------------------
# exchange through symmetric memory (in-tree peer-memory kernels), with torch.distributed as the other path
# ---------------------------------------------------------------------------------------------------------------
_WS = {}


def _workspace(tag: str, numel: int, dtype, device):
    """A symmetric flat tensor of at least ``numel`` elements for the CP group (grown by re-allocation: collective)."""
    from . import dp_comm
    key = (tag, dtype, tuple(ps.get_group_ranks('cp')))      # a workspace belongs to one set of peers
    cur = _WS.get(key)
    if cur is None or cur[1].numel() < numel:
        if cur is not None:
            torch.cuda.synchronize()
        ws, flat = dp_comm.allocate('cp', numel, dtype)
        _WS[key] = cur = (ws, flat)
    return cur


def _fused_exchange(device) -> bool:
    from . import dp_comm
    return dp_comm.usable('cp', device)


def _all_gather_kv(k: torch.Tensor, v: torch.Tensor):
    """``k`` / ``v`` ``[T_local, nkv, d]`` of every rank -> rank-major ``[cp * T_local, nkv, d]`` pair."""
    cp, r = ps.get_world_size('cp'), ps.get_rank_in('cp')
    tl = k.shape[0]
    per = k[0].numel() + v[0].numel()          # elements of one token's K and V
    if _fused_exchange(k.device):
        from . import dp_comm
        n = tl * per
        ws, flat = _workspace('kv', cp * n, k.dtype, k.device)
        mine = flat[r * n:(r + 1) * n]
        mine[:tl * k[0].numel()].view_as(k).copy_(k)
        mine[tl * k[0].numel():].view_as(v).copy_(v)
        dp_comm.all_gather_(ws, flat, 0, cp * n)
        slots = flat[:cp * n].view(cp, n)
        kg = slots[:, :tl * k[0].numel()].reshape(cp * tl, *k.shape[1:])
        vg = slots[:, tl * k[0].numel():].reshape(cp * tl, *v.shape[1:])
        return kg, vg
    group = ps.get_group('cp')
    kg = torch.empty((cp * tl, *k.shape[1:]), dtype=k.dtype, device=k.device)
    vg = torch.empty((cp * tl, *v.shape[1:]), dtype=v.dtype, device=v.device)
    dist.all_gather_into_tensor(kg, k.contiguous(), group=group)
    dist.all_gather_into_tensor(vg, v.contiguous(), group=group)
    return kg, vg


def _reduce_scatter_kv_grads(dk_rm: torch.Tensor, dv_rm: torch.Tensor, dtype):
    """Rank-major gradients of all keys / values on every rank -> this rank's slice of their sum (fp32 accumulation)."""
    cp, r = ps.get_world_size('cp'), ps.get_rank_in('cp')
    tl = dk_rm.shape[0] // cp
    nk, nv = dk_rm[0].numel(), dv_rm[0].numel()
    if _fused_exchange(dk_rm.device):
        from . import dp_comm
        n = tl * (nk + nv)
        ws, flat = _workspace('dkv', cp * n, torch.float32, dk_rm.device)
        slots = flat[:cp * n].view(cp, n)
        slots[:, :tl * nk].copy_(dk_rm.reshape(cp, tl * nk))
        slots[:, tl * nk:].copy_(dv_rm.reshape(cp, tl * nv))
        dp_comm.reduce_scatter_(ws, flat, 0, cp * n, 1.0)
        mine = flat[r * n:(r + 1) * n]
        dk = mine[:tl * nk].view(tl, *dk_rm.shape[1:]).to(dtype)
        dv = mine[tl * nk:].view(tl, *dv_rm.shape[1:]).to(dtype)
        return dk, dv
    group = ps.get_group('cp')
    dk = torch.empty((tl, *dk_rm.shape[1:]), dtype=torch.float32, device=dk_rm.device)
    dv = torch.empty((tl, *dv_rm.shape[1:]), dtype=torch.float32, device=dv_rm.device)
    dist.reduce_scatter_tensor(dk, dk_rm.float().contiguous(), group=group)
    dist.reduce_scatter_tensor(dv, dv_rm.float().contiguous(), group=group)
    return dk.to(dtype), dv.to(dtype)


class _GatherKV(torch.autograd.Function):
    """``(k, v)`` of this rank -> rank-major ``(k, v)`` of all ranks; backward returns to every rank the summed
    gradients of its own rows.  Both directions run on the peer-memory kernels when the group supports them."""

    @staticmethod
    def forward(ctx, k, v):
        ctx.kv_dtype = k.dtype
        kg, vg = _all_gather_kv(k, v)
        # the gathered rows live in a workspace the next call reuses: hand out copies
        return kg.clone(), vg.clone()

    @staticmethod
    def backward(ctx, dkg, dvg):
        return _reduce_scatter_kv_grads(dkg, dvg, ctx.kv_dtype)


def gather_to_stream_order(x: torch.Tensor, ctx) -> torch.Tensor:
    """``[T_local, ...]`` on every CP rank -> ``[cp * T_local, ...]`` in the order of the original token stream
    (differentiable: the backward reduce-scatters)."""
    lay = get_layout(ctx, x.shape[0], x.device)
    return _AllGatherTokens.apply(x, 'cp').index_select(0, lay.gather_index)


def stream_index_of_local_tokens(ctx, device, t_local: Optional[int] = None) -> torch.Tensor:
    """Position in the original token stream of every token this CP rank holds, in local order."""
    if t_local is None:
        cu = ctx.cu_seqlens
        assert cu is not None, 'pass t_local when the batch is not packed'
        lay = ctx.extra.get('cp_layout')
        assert lay is not None, 'the layout is created by the first cp_attention / gather_to_stream_order call'
        return lay.q_stream
    return get_layout(ctx, t_local, device).q_stream


# ---------------------------------------------------------------------------------------------------------------
# ring form (cp_comm_type = 'p2p'): one chunk of keys / values per step, the next chunk fetched behind the kernel
# ---------------------------------------------------------------------------------------------------------------
def _range_mask(lo: torch.Tensor, hi: torch.Tensor, tk: int) -> torch.Tensor:
    pos = torch.arange(tk, device=lo.device)[None, :]
    return (pos >= lo[:, None].long()) & (pos <= hi[:, None].long())        # [T, Tk]


def _partial_fwd_ref(q, k, v, lo, hi, scale):
    """fp32 attention of every query over its key range in this chunk -> (o [T, nq, d] un-normalised by nothing:
    softmax within the chunk, lse [nq, T]); rows with an empty range give o = 0, lse = -inf."""
    nq, nkv = q.shape[1], k.shape[1]
    kf = k.float().repeat_interleave(nq // nkv, dim=1)
    vf = v.float().repeat_interleave(nq // nkv, dim=1)
    sc = torch.einsum('ihd,jhd->hij', q.float(), kf) * scale
    sc = sc.masked_fill(~_range_mask(lo, hi, k.shape[0])[None], float('-inf'))
    lse = torch.logsumexp(sc, dim=-1)
    p = torch.exp(sc - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    return torch.einsum('hij,jhd->ihd', p, vf), lse


def _partial_bwd_ref(q, k, v, do, lse, delta, lo, hi, scale):
    """Gradients of one chunk given the final log-sum-exp and delta = rowsum(o * do): (dq, dk, dv) in fp32."""
    nq, nkv = q.shape[1], k.shape[1]
    g = nq // nkv
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    sc = torch.einsum('ihd,jhd->hij', q.float(), kf) * scale
    p = torch.exp(sc - lse[..., None]).masked_fill(~_range_mask(lo, hi, k.shape[0])[None], 0.0)
    dof = do.float()
    dv = torch.einsum('hij,ihd->jhd', p, dof)
    ds = p * (torch.einsum('ihd,jhd->hij', dof, vf) - delta[..., None]) * scale
    dq = torch.einsum('hij,jhd->ihd', ds, kf)
    dk = torch.einsum('hij,ihd->jhd', ds, q.float())
    tk = k.shape[0]
    return dq, dk.view(tk, nkv, g, -1).sum(2), dv.view(tk, nkv, g, -1).sum(2)


class _ChunkFetcher:
    """Hands out the keys / values of the CP ranks one chunk at a time.  On a GPU with peer-mapped memory every rank
    publishes its K / V in a symmetric buffer and the copy engine pulls the next rank's chunk on a side stream while
    the attention kernel works on the current one; elsewhere the chunks come from one ``torch.distributed``
    all-gather."""

    _side = {}
    _epoch = 0

    def __init__(self, k: torch.Tensor, v: torch.Tensor):
        self.cp, self.rank = ps.get_world_size('cp'), ps.get_rank_in('cp')
        self.k, self.v = k.contiguous(), v.contiguous()
        self.nk, self.nv = self.k.numel(), self.v.numel()
        self.peer = _fused_exchange(k.device)
        self.pending = None
        if self.peer:
            n = self.nk + self.nv
            _ChunkFetcher._epoch += 1
            self.base = (_ChunkFetcher._epoch & 1) * n        # two halves: a rank republishes only two calls later
            self.ws, flat = _workspace('ring_kv', 2 * n, k.dtype, k.device)
            mine = flat[self.base:self.base + n]
            mine[:self.nk].view_as(self.k).copy_(self.k)
            mine[self.nk:].view_as(self.v).copy_(self.v)
            self.ws.handle.barrier(channel=0)                  # every rank's chunk is in place (stream-ordered)
            dev = k.device.index
            if dev not in _ChunkFetcher._side:
                _ChunkFetcher._side[dev] = torch.cuda.Stream(device=k.device)
            self.side = _ChunkFetcher._side[dev]
            self.published = torch.cuda.Event()
            self.published.record()
        else:
            group = ps.get_group('cp')
            self.kg = torch.empty((self.cp, *self.k.shape), dtype=k.dtype, device=k.device)
            self.vg = torch.empty((self.cp, *self.v.shape), dtype=v.dtype, device=v.device)
            dist.all_gather_into_tensor(self.kg.view(-1, *self.k.shape[1:]), self.k, group=group)
            dist.all_gather_into_tensor(self.vg.view(-1, *self.v.shape[1:]), self.v, group=group)

    def prefetch(self, j: int):
        """Starts bringing rank ``j``'s chunk into local memory (no-op for the own chunk and off the peer path)."""
        if not self.peer or j == self.rank:
            return
        from .dp_comm import FLAG_BYTES
        n = self.nk + self.nv
        es = self.k.element_size()
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.side):
            self.side.wait_event(self.published)
            buf = torch.empty(n, dtype=self.k.dtype, device=self.k.device)
            src = self.ws.handle.get_buffer(j, (n,), self.k.dtype, FLAG_BYTES // es + self.base)
            buf.copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        buf.record_stream(main)
        self.pending = (j, buf, ev)

    def get(self, j: int):
        if j == self.rank:
            return self.k, self.v
        if not self.peer:
            return self.kg[j], self.vg[j]
        if self.pending is None or self.pending[0] != j:
            self.prefetch(j)
        _, buf, ev = self.pending
        self.pending = None
        torch.cuda.current_stream().wait_event(ev)
        return buf[:self.nk].view_as(self.k), buf[self.nk:].view_as(self.v)


class _RingAttnFn(torch.autograd.Function):
    """Context-parallel attention one source rank at a time: step ``s`` attends to the keys / values of rank
    ``(r - s) mod cp`` (a contiguous range of that rank's tokens per query, ``CpLayout.ring_lo / ring_hi``) while the
    next rank's chunk is on its way; the partial results are merged through their log-sum-exp.  Only the local K / V
    are kept for the backward pass, which fetches the chunks again, recomputes the probabilities from the final
    log-sum-exp and returns the key / value gradients through the reduce-scatter of the all-gather form."""

    @staticmethod
    def forward(ctx, q, k, v, lay: CpLayout, scale: float, use_kernel: bool):
        cp, r = lay.cp, lay.rank
        T, nq, d = q.shape
        fetch = _ChunkFetcher(k, v)
        o_acc = torch.zeros((T, nq, v.shape[-1]), dtype=torch.float32, device=q.device)
        lse_acc = torch.full((nq, T), float('-inf'), dtype=torch.float32, device=q.device)
        qc = q.contiguous()
        for s in range(cp):
            j = (r - s) % cp
            if s + 1 < cp:
                fetch.prefetch((r - s - 1) % cp)
            kj, vj = fetch.get(j) if s else (fetch.k, fetch.v)
            if use_kernel:
                from ..ops import attention_cuda as ac
                o_s, lse_s = ac.fwd_ranges_raw(qc, kj, vj, lay.ring_lo[j], lay.ring_hi[j], scale)
                o_s = o_s.float()
            else:
                o_s, lse_s = _partial_fwd_ref(qc, kj, vj, lay.ring_lo[j], lay.ring_hi[j], scale)
            new = torch.logaddexp(lse_acc, lse_s)
            safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
            w_old = torch.exp(lse_acc - safe).t()[..., None]       # exp(-inf) = 0 for rows that had nothing yet
            w_new = torch.exp(lse_s - safe).t()[..., None]
            o_acc = o_acc * w_old + o_s * w_new
            lse_acc = new
        o = o_acc.to(q.dtype)
        ctx.save_for_backward(qc, fetch.k, fetch.v, o, lse_acc)
        ctx.lay, ctx.scale, ctx.use_kernel = lay, scale, use_kernel
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        lay, scale = ctx.lay, ctx.scale
        cp, r = lay.cp, lay.rank
        do = do.contiguous()
        delta = (o.float() * do.float()).sum(-1).t().contiguous()              # [nq, T]
        fetch = _ChunkFetcher(k, v)
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dk_rm = torch.empty((cp, *k.shape), dtype=torch.float32, device=q.device)
        dv_rm = torch.empty((cp, *v.shape), dtype=torch.float32, device=q.device)
        for s in range(cp):
            j = (r - s) % cp
            if s + 1 < cp:
                fetch.prefetch((r - s - 1) % cp)
            kj, vj = fetch.get(j) if s else (fetch.k, fetch.v)
            if ctx.use_kernel:
                from ..ops import attention_cuda as ac
                dq_s, dk_s, dv_s = ac.bwd_ranges_raw(q, kj, vj, o, do, lse, delta, lay.ring_lo[j], lay.ring_hi[j],
                                                     lay.ring_qlo[j], lay.ring_qhi[j], scale)
            else:
                dq_s, dk_s, dv_s = _partial_bwd_ref(q, kj, vj, do, lse, delta, lay.ring_lo[j], lay.ring_hi[j], scale)
            dq += dq_s.float()
            dk_rm[j].copy_(dk_s)
            dv_rm[j].copy_(dv_s)
        dk, dv = _reduce_scatter_kv_grads(dk_rm.view(-1, *k.shape[1:]), dv_rm.view(-1, *v.shape[1:]), k.dtype)
        return dq.to(q.dtype), dk, dv, None, None, None


def cp_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx, scale: Optional[float] = None,
                 window=None, sinks=None, comm_type: Optional[str] = None) -> torch.Tensor:
    """``q/k/v`` hold this rank's tokens ``[T_local, heads, d]``; returns ``[T_local, nq, dv]``.  ``comm_type`` is the
    layer's ``cp_comm_type``: ``'p2p'`` (the reference's default) runs the ring form, anything else (``'allgather'``,
    ``'a2a'``, ...) the all-gather form; masks the ring does not cover (window, sinks) use the all-gather form."""
    lay = get_layout(ctx, q.shape[0], q.device)
    from ..ops import attention_cuda as ac
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if (comm_type or 'p2p') == 'p2p' and window is None and sinks is None and k.shape[-1] == v.shape[-1]:
        kernel = ac.ranges_supported(q, k, v)
        if kernel or not q.is_cuda:
            return _RingAttnFn.apply(q, k, v, lay, float(scale), kernel)
    if window is None and sinks is None and ac.ranges_supported(q, k, v):
        kg, vg = _GatherKV.apply(k, v)
        k_full, v_full = kg.index_select(0, lay.gather_index), vg.index_select(0, lay.gather_index)
        o, _ = ac.attention_ranges(q, k_full, v_full, lay.k_lo, lay.k_hi, lay.q_lo, lay.q_hi, scale)
        return o
    if q.is_cuda:
        from ..ops import _lib
        if _lib.cuda_enabled():
            from ..utils.logger import get_logger
            get_logger().warning_once('context-parallel attention: head size / mask option outside the in-tree kernel; '
                                      'keys and values are all-gathered with torch.distributed and the generic '
                                      'attention op runs')
    k_full = _AllGatherTokens.apply(k, 'cp').index_select(0, lay.gather_index)
    v_full = _AllGatherTokens.apply(v, 'cp').index_select(0, lay.gather_index)
    from ..ops.attention import attention_qk_ranges
    return attention_qk_ranges(q, k_full, v_full, lay, scale, window, sinks)


# kept under the name earlier call sites import
ring_attention = cp_attention
