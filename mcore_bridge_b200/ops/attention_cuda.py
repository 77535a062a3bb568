"""Binding of the in-tree sm_100a attention kernels (filled in as the kernels land)."""
from __future__ import annotations

import torch


def supported(q, k, v, causal, window, sinks, softcap) -> bool:
    return False


def attention(q, k, v, cu_seqlens, max_seqlen, scale):
    raise NotImplementedError
