"""ctypes loader for the in-tree CUDA library ``lib/libmcb200.so``.

The library is built by :mod:`mcore_bridge_b200.build_ext`.  On a machine with a GPU a missing
library is an error (ops must not fall back silently to PyTorch there); on a CPU-only machine
:func:`available` is simply False and the torch reference implementations are used.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / 'lib' / 'libmcb200.so'
_lib = None
_lock = threading.Lock()
_status_words: dict[int, torch.Tensor] = {}
LAUNCHES = 0  # kernel launches issued through this library (every op reports exactly one per launch)

STATUS_NAMES = {
    0: 'ok', 1: 'timeout waiting for a filled smem stage', 2: 'timeout waiting for a free smem stage',
    3: 'timeout waiting for a full TMEM accumulator', 4: 'timeout waiting for a free TMEM accumulator',
    5: 'timeout waiting for a peer flag', 6: 'bad argument', 7: 'MoE receive buffer too small for this routing',
}
ST_MOE_OVERFLOW = 7


class KernelError(RuntimeError):
    pass


def cuda_enabled() -> bool:
    """True when the hand-written kernels should be used (a CUDA device is present and not disabled)."""
    return torch.cuda.is_available() and os.environ.get('MCB200_DISABLE_CUDA_KERNELS', '0') != '1'


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not _LIB_PATH.exists():
                    if torch.cuda.is_available():
                        from ..build_ext import build
                        build(verbose=False)
                    if not _LIB_PATH.exists():
                        raise KernelError(f'{_LIB_PATH} is missing: run `python -m mcore_bridge_b200.build_ext`')
                _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


def available() -> bool:
    if not cuda_enabled():
        return False
    lib()  # raises loudly on a GPU box without the library
    return True


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 status word the kernels write when a bounded wait gives up."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    w = _status_words.get(dev)
    if w is None:
        w = torch.zeros(16, dtype=torch.int32, device=f'cuda:{dev}')
        w[1] = int(os.environ.get('MCB200_WAIT_LIMIT_MS', '10000'))  # bound of every in-kernel wait
        _status_words[dev] = w
    return w


def check_status(device=None, clear: bool = True) -> None:
    """Synchronising check of the status word; raises :class:`KernelError` if a kernel gave up a wait."""
    w = status_word(device)
    code = int(w[0].item())
    if code != 0:
        if clear:
            w[0] = 0
        raise KernelError(f'kernel status {code}: {STATUS_NAMES.get(code, "unknown")}')


def check_rc(rc: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise KernelError(f'{what} failed with code {rc}' + (' (CUDA error)' if rc > 0 else ' (bad argument)'))
