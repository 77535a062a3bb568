"""MoE routing and token permutation.

* :func:`topk_routing` — softmax / sigmoid scores, group-limited selection, expert bias, top-k scaling,
  pre-/post-softmax normalisation; fp32 throughout (``moe_router_dtype='fp32'``).
* :func:`aux_loss` / :func:`seq_aux_loss` — load-balancing losses; :class:`MoEAuxLossAutoScaler` attaches
  them to the activation so they reach the router through the normal backward pass.
* :func:`permute` / :func:`unpermute` — sort (token, choice) pairs by expert into a buffer whose per-expert
  segments are padded to 128 rows (the tile height of the grouped GEMM); every size is static and the
  offsets stay on the device, so nothing synchronises with the host.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

PAD = 128


def topk_routing(logits: torch.Tensor, topk: int, score_function: str = 'softmax', pre_softmax: bool = False,
                 num_groups: Optional[int] = None, group_topk: Optional[int] = None,
                 scaling_factor: Optional[float] = None, expert_bias: Optional[torch.Tensor] = None,
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``(probs [T, k], indices [T, k], scores [T, E])``; ``scores`` feed the auxiliary loss.

    softmax + ``pre_softmax``: softmax over all experts, pick top-k, keep the raw probabilities.
    softmax otherwise: pick top-k logits, softmax over the selected k (= renormalised probabilities).
    sigmoid: scores = sigmoid(logits); selection uses ``scores + expert_bias`` when a bias is given; the
    selected scores are normalised to sum to one (when k > 1 and not ``pre_softmax``), then scaled.
    """
    logits = logits.float()
    T, E = logits.shape

    def select(sel_scores):
        if num_groups is not None and num_groups > 1 and group_topk is not None:
            g = sel_scores.view(T, num_groups, E // num_groups)
            # group score: sum of its top (topk / group_topk) entries
            per = max(1, topk // group_topk)
            gscore = g.topk(min(per, g.shape[-1]), dim=-1).values.sum(-1)
            gidx = gscore.topk(group_topk, dim=-1).indices
            gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, gidx, True)
            masked = sel_scores.masked_fill(~gmask[:, :, None].expand_as(g).reshape(T, E), float('-inf'))
            return masked.topk(topk, dim=-1).indices
        return sel_scores.topk(topk, dim=-1).indices

    if score_function == 'softmax':
        if expert_bias is not None:
            # Ernie-4.5: the probabilities plus a correction bias pick the experts, the weights are the picked
            # probabilities (renormalised unless ``pre_softmax``)
            scores = torch.softmax(logits, dim=-1)
            idx = select(scores + expert_bias.float())
            probs = scores.gather(1, idx)
            if not pre_softmax:
                probs = probs / probs.sum(-1, keepdim=True).clamp(min=1e-12)
        elif pre_softmax:
            scores = torch.softmax(logits, dim=-1)
            idx = select(scores)
            probs = scores.gather(1, idx)
        else:
            idx = select(logits)
            probs = torch.softmax(logits.gather(1, idx), dim=-1)
            scores = torch.softmax(logits, dim=-1)
    elif score_function == 'sigmoid':
        scores = torch.sigmoid(logits)
        idx = select(scores + expert_bias.float() if expert_bias is not None else scores)
        probs = scores.gather(1, idx)
        if topk > 1 and not pre_softmax:        # ``pre_softmax`` here: keep the raw scores (``norm_topk_prob=False``)
            probs = probs / (probs.sum(-1, keepdim=True) + 1e-20)
    else:
        raise ValueError(f'unknown score function {score_function}')
    if scaling_factor:
        probs = probs * scaling_factor
    return probs, idx, scores


def tokens_per_expert(indices: torch.Tensor, num_experts: int, valid: Optional[torch.Tensor] = None) -> torch.Tensor:
    flat = indices.reshape(-1)
    if valid is not None:
        w = valid.reshape(-1, 1).expand_as(indices).reshape(-1).to(torch.float32)
        return torch.zeros(num_experts, device=indices.device, dtype=torch.float32).index_add_(0, flat, w)
    return torch.bincount(flat, minlength=num_experts).float()


def aux_loss(scores: torch.Tensor, counts: torch.Tensor, topk: int, coeff: float, num_tokens) -> torch.Tensor:
    """Switch-style load-balancing loss ``coeff * E * sum_e f_e * P_e`` with ``f_e`` the routed fraction
    and ``P_e`` the mean score; ``counts``/``num_tokens`` may be pre-reduced over a group."""
    E = scores.shape[-1]
    mean_scores = scores.sum(0) / num_tokens
    frac = counts / (num_tokens * topk)
    return coeff * E * (frac * mean_scores).sum()


def seq_aux_loss(scores: torch.Tensor, indices: torch.Tensor, seg_ids: torch.Tensor, num_seqs: int, topk: int,
                 coeff: float, group=None) -> torch.Tensor:
    """Per-sequence load-balancing loss (DeepSeek): the loss above computed inside each packed sequence,
    averaged over sequences.  Scores are normalised over experts first.

    ``group``: process group whose ranks each hold part of every sequence (sequence / context parallelism).  The
    selection counts and sequence lengths are then summed over it and this rank's term uses its own share of the
    mean probability, so the ranks' values add up to the loss of the whole sequences."""
    T, E = scores.shape
    sn = scores / (scores.sum(-1, keepdim=True) + 1e-20)
    onehot = torch.zeros(T, E, device=scores.device, dtype=torch.float32).scatter_add_(
        1, indices, torch.ones_like(indices, dtype=torch.float32))
    lens = torch.bincount(seg_ids, minlength=num_seqs).float()
    cnt = torch.zeros(num_seqs, E, device=scores.device).index_add_(0, seg_ids, onehot)
    if group is not None:
        packed = torch.cat([cnt, lens[:, None]], dim=1)
        torch.distributed.all_reduce(packed, group=group)
        cnt, lens = packed[:, :E], packed[:, E]
    lens = lens.clamp(min=1)
    sm = torch.zeros(num_seqs, E, device=scores.device).index_add_(0, seg_ids, sn)
    f = cnt * E / (topk * lens[:, None])
    p = sm / lens[:, None]
    return coeff * (f * p).sum(-1).mean()


class MoEAuxLossAutoScaler(torch.autograd.Function):
    """Identity on the activation; in backward injects d(aux_loss) = loss_scale so the router gets its gradient
    without the aux loss being part of the returned language-model loss."""
    main_loss_backward_scale: float = 1.0

    @staticmethod
    def forward(ctx, output, aux):
        ctx.save_for_backward(aux)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (aux,) = ctx.saved_tensors
        return grad_output, torch.ones_like(aux) * MoEAuxLossAutoScaler.main_loss_backward_scale

    @staticmethod
    def set_loss_scale(scale: float):
        MoEAuxLossAutoScaler.main_loss_backward_scale = float(scale)


def z_loss(logits: torch.Tensor, coeff: float) -> torch.Tensor:
    return coeff * torch.logsumexp(logits.float(), dim=-1).square().mean()


# ------------------------------------------------------------------ permutation
def padded_capacity(num_items: int, num_experts: int, pad: int = PAD) -> int:
    """Static row count that always fits ``num_items`` rows split over ``num_experts`` padded segments."""
    return ((num_items + num_experts * (pad - 1)) + pad - 1) // pad * pad


def permute_plan(expert_ids: torch.Tensor, num_experts: int, pad: int = PAD, capacity: Optional[int] = None):
    """``expert_ids [M]`` (one per routed copy) -> ``(dest_row [M], offsets [E+1] int32, capacity)``.

    ``dest_row[i]`` is the row of copy ``i`` in the expert-sorted padded buffer; segment ``e`` is
    ``offsets[e]:offsets[e+1]`` and holds its copies first, zero rows after.
    """
    M = expert_ids.numel()
    flat = expert_ids.reshape(-1).to(torch.int64)
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + pad - 1) // pad * pad
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    offsets[1:] = padded.cumsum(0)
    order = torch.argsort(flat, stable=True)
    starts = torch.zeros(num_experts, dtype=torch.int64, device=flat.device)
    starts[1:] = counts.cumsum(0)[:-1]
    sorted_e = flat[order]
    pos = torch.arange(M, device=flat.device) - starts[sorted_e]
    dest_sorted = offsets[:-1][sorted_e] + pos
    dest = torch.empty(M, dtype=torch.int64, device=flat.device)
    dest[order] = dest_sorted
    cap = capacity if capacity is not None else padded_capacity(M, num_experts, pad)
    return dest, offsets.to(torch.int32), cap


class _Permute(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, src_token, dest_row, capacity):
        out = torch.zeros((capacity, x.shape[-1]), dtype=x.dtype, device=x.device)
        out.index_copy_(0, dest_row, x.index_select(0, src_token))
        ctx.save_for_backward(src_token, dest_row)
        ctx.n = x.shape[0]
        return out

    @staticmethod
    def backward(ctx, g):
        src_token, dest_row = ctx.saved_tensors
        dx = torch.zeros((ctx.n, g.shape[-1]), dtype=torch.float32, device=g.device)
        dx.index_add_(0, src_token, g.index_select(0, dest_row).float())
        return dx.to(g.dtype), None, None, None


def permute(x: torch.Tensor, src_token: torch.Tensor, dest_row: torch.Tensor, capacity: int) -> torch.Tensor:
    """Row ``dest_row[i]`` of the result is ``x[src_token[i]]``; all other rows are zero."""
    return _Permute.apply(x, src_token, dest_row, capacity)


class _Unpermute(torch.autograd.Function):

    @staticmethod
    def forward(ctx, y, src_token, dest_row, num_tokens, probs):
        rows = y.index_select(0, dest_row).float()
        if probs is not None:
            rows = rows * probs.reshape(-1, 1).float()
        out = torch.zeros((num_tokens, y.shape[-1]), dtype=torch.float32, device=y.device)
        out.index_add_(0, src_token, rows)
        ctx.save_for_backward(src_token, dest_row, probs, y if probs is not None else None)
        ctx.cap = y.shape[0]
        return out.to(y.dtype)

    @staticmethod
    def backward(ctx, g):
        src_token, dest_row, probs, y = ctx.saved_tensors
        grows = g.index_select(0, src_token)
        dprobs = None
        if probs is not None:
            dprobs = (grows.float() * y.index_select(0, dest_row).float()).sum(-1).view(probs.shape).to(probs.dtype)
            grows = (grows.float() * probs.reshape(-1, 1).float()).to(g.dtype)
        dy = torch.zeros((ctx.cap, g.shape[-1]), dtype=g.dtype, device=g.device)
        dy.index_copy_(0, dest_row, grows)
        return dy, None, None, None, dprobs


def unpermute(y: torch.Tensor, src_token: torch.Tensor, dest_row: torch.Tensor, num_tokens: int,
              probs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum_{i: src_token[i]==t} probs[i] * y[dest_row[i]]``."""
    return _Unpermute.apply(y, src_token, dest_row, num_tokens, probs)
