"""The allocation-free RMSNorm backward (``mcb_rmsnorm_bwd_noalloc``), called through its exported C symbol.

Some callers of the library cannot allocate device memory at the point where they need a kernel: a callback running
inside another component's stream-ordered region, a process whose memory was carved up front, a thread that must not
touch the allocator.  For them the library keeps the kernel's fp32 weight-gradient accumulator in a fixed device
array.  This test drives that entry point with caller-owned buffers only and checks it against the regular entry
point (which gets its accumulator from the caller) on two consecutive calls — the second one proves that the shared
array is cleared between calls.  It lives in the file pytest collects last so that a failure here cannot hide the
result of any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_pair(lib, rows, H, zero_centered, seed):
    from mcore_bridge_b200.ops import _lib
    torch.manual_seed(seed)
    dev = 'cuda'
    x = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    w = (torch.randn(H, device=dev) * 0.1 + (0.0 if zero_centered else 1.0)).to(torch.bfloat16)
    ll, i32, f32 = ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    stream = _lib.stream_ptr()
    # regular entry point: the caller supplies the fp32 accumulator
    dx_ref = torch.empty_like(x)
    dw_acc = torch.zeros(H, dtype=torch.float32, device=dev)
    rc = lib.mcb_rmsnorm_bwd(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(w), None, None, _lib.ptr(dx_ref), _lib.ptr(dw_acc),
                             ll(rows), i32(H), ll(H), f32(1e-6), i32(int(zero_centered)), stream)
    assert rc == 0
    # allocation-free entry point: outputs only
    dx = torch.empty_like(x)
    dw = torch.empty(H, dtype=torch.bfloat16, device=dev)
    rc = lib.mcb_rmsnorm_bwd_noalloc(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(dx), _lib.ptr(dw), ll(rows),
                                     i32(H), ll(H), f32(1e-6), i32(int(zero_centered)), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dx, dx_ref)
    ref = dw_acc
    err = (dw.float() - ref).norm() / ref.norm()
    assert err.item() < 1e-2, err.item()   # bf16 rounding of the result + fp32 atomic summation order


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    from mcore_bridge_b200.ops import _lib
    assert _lib.available()
    lib = _lib.lib()
    lib.mcb_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    _run_pair(lib, 1000, 4096, False, 1)
    _run_pair(lib, 333, 2048, True, 2)     # smaller H after a larger one: stale sums beyond H must not matter


def test_noalloc_rejects_oversized_hidden():
    from mcore_bridge_b200.ops import _lib
    lib = _lib.lib()
    rc = lib.mcb_rmsnorm_bwd_noalloc(None, None, None, None, None, ctypes.c_longlong(1), ctypes.c_int(16384 + 8),
                                     ctypes.c_longlong(16392), ctypes.c_float(1e-6), ctypes.c_int(0), None)
    assert rc == -20
