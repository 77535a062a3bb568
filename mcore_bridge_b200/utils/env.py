"""Rank / world-size helpers read from the launcher's environment (``torchrun`` variables).

Parity: reference ``src/mcore_bridge/utils/env.py:12-50``.
"""
from __future__ import annotations

import os
from typing import Tuple


def use_hf_hub() -> bool:
    return os.environ.get('USE_HF', '0').lower() in {'1', 'true'}


def get_dist_setting() -> Tuple[int, int, int, int]:
    """(rank, local_rank, world_size, local_world_size); -1 / 1 when not launched distributed."""
    rank = int(os.getenv('RANK', -1))
    local_rank = int(os.getenv('LOCAL_RANK', -1))
    world_size = int(os.getenv('WORLD_SIZE') or os.getenv('_PATCH_WORLD_SIZE') or 1)
    local_world_size = int(os.getenv('LOCAL_WORLD_SIZE', None) or os.getenv('LOCAL_SIZE', 1))
    return rank, local_rank, world_size, local_world_size


def get_node_setting() -> Tuple[int, int]:
    return int(os.getenv('NODE_RANK', 0)), int(os.getenv('NNODES', 1))


def is_local_master() -> bool:
    return get_dist_setting()[1] in {-1, 0}


def is_master() -> bool:
    return get_dist_setting()[0] in {-1, 0}


def is_last_rank() -> bool:
    rank, _, world_size, _ = get_dist_setting()
    return rank in {-1, world_size - 1}


def is_dist() -> bool:
    rank, local_rank, _, _ = get_dist_setting()
    return rank >= 0 and local_rank >= 0
