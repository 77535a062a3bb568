"""Device / synchronisation helpers (parity: reference ``src/mcore_bridge/utils/torch_utils.py:28-161``)."""
from __future__ import annotations

import gc
import hashlib
import os
import time
from contextlib import contextmanager
from typing import Any, Mapping, Optional, Union

import torch
import torch.distributed as dist

from .env import get_dist_setting, is_dist, is_local_master


def synchronize(device=None):
    if torch.cuda.is_available():
        torch.cuda.synchronize(device)


def time_synchronize() -> float:
    synchronize()
    return time.perf_counter()


@contextmanager
def safe_ddp_context(hash_id: Optional[str], use_barrier: bool = True):
    """Lets the (local) master run the body first — e.g. a download or a cache build — then the others.

    With ``use_barrier`` and an initialised process group this is two barriers; otherwise a lock file
    keyed by ``hash_id`` serialises the processes of one node.
    """
    if use_barrier and dist.is_available() and dist.is_initialized():
        master = (is_dist() and is_local_master()) or not is_dist()
        if not master:
            dist.barrier()
        yield
        if master:
            dist.barrier()
        return
    if hash_id is None:
        yield
        return
    lock_dir = os.path.join(os.path.expanduser('~'), '.cache', 'mcore_bridge_b200', 'locks')
    os.makedirs(lock_dir, exist_ok=True)
    path = os.path.join(lock_dir, hashlib.sha256(hash_id.encode()).hexdigest() + '.lock')
    from filelock import FileLock
    with FileLock(path):
        yield


def get_device(local_rank: Optional[Union[str, int]] = None) -> str:
    if local_rank is None:
        local_rank = max(0, get_dist_setting()[1])
    return f'cuda:{local_rank}' if torch.cuda.is_available() else 'cpu'


def get_current_device():
    if torch.cuda.is_available():
        return torch.device('cuda', torch.cuda.current_device())
    return torch.device('cpu')


def get_torch_device():
    return torch.cuda if torch.cuda.is_available() else torch.cpu


def set_device(local_rank: Optional[Union[str, int]] = None):
    if torch.cuda.is_available():
        if local_rank is None:
            local_rank = max(0, get_dist_setting()[1])
        torch.cuda.set_device(int(local_rank))


def get_device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def empty_cache():
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def gc_collect() -> None:
    gc.collect()
    empty_cache()


def to_float_dtype(data: Any, dtype: torch.dtype) -> Any:
    if isinstance(data, Mapping):
        return type(data)({k: to_float_dtype(v, dtype) for k, v in data.items()})
    if isinstance(data, (tuple, list)):
        return type(data)(to_float_dtype(v, dtype) for v in data)
    if isinstance(data, torch.Tensor) and torch.is_floating_point(data):
        return data.to(dtype=dtype)
    return data


def to_device(data: Any, device, non_blocking: bool = False) -> Any:
    if isinstance(data, Mapping):
        return type(data)({k: to_device(v, device, non_blocking) for k, v in data.items()})
    if isinstance(data, (tuple, list)):
        return type(data)(to_device(v, device, non_blocking) for v in data)
    if isinstance(data, torch.Tensor):
        return data.to(device=device, non_blocking=non_blocking)
    return data


def host_list(t: torch.Tensor):
    """Values of a small integer tensor (sequence boundaries) as a Python list.  A device tensor that was copied from
    host memory can carry the host values in ``_host_list`` (:func:`attach_host_list`); reading them from there does
    not wait for the device, ``tolist()`` on a device tensor does."""
    cached = getattr(t, '_host_list', None)
    if cached is not None:
        return list(cached)
    return [int(x) for x in t.tolist()]


def attach_host_list(device_tensor: torch.Tensor, host_tensor: torch.Tensor) -> torch.Tensor:
    """Remember the values of ``host_tensor`` on its device copy (see :func:`host_list`)."""
    if host_tensor.device.type == 'cpu' and host_tensor.numel() <= 1 << 16:
        device_tensor._host_list = tuple(int(x) for x in host_tensor.tolist())
    return device_tensor

