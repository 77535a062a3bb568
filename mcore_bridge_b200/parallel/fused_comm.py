"""Fused compute+collective kernels over NVLink peer memory (filled in as the kernels land).

``enabled`` gates every call site in ``ops/linear.py``; while it answers False the
``torch.distributed`` path runs.
"""
from __future__ import annotations


def enabled(x, weight, group_name: str) -> bool:
    return False
