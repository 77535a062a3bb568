"""Builds the CUDA sources under ``csrc/`` into one in-tree shared library for sm_100a.

The kernels expose a plain C ABI and are loaded through ``ctypes`` (see ``ops/_lib.py``), so the
build is a handful of ``nvcc`` invocations with no dependency on the torch headers: a full
rebuild takes seconds and works on a machine without a GPU (nvcc cross-compiles).

Run as ``python -m mcore_bridge_b200.build_ext`` or call :func:`build`.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = REPO_DIR / 'csrc'
LIB_DIR = PKG_DIR / 'lib'
LIB_NAME = 'libmcb200.so'
OBJ_DIR = REPO_DIR / 'build' / 'obj'

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '--use_fast_math',
    '-Xcompiler', '-fPIC', '-Xptxas', '-v', '--expt-relaxed-constexpr',
]


def _nvcc() -> str:
    cand = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(cand):
        raise RuntimeError('nvcc not found; the CUDA kernels of mcore_bridge_b200 cannot be built')
    return cand


def sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob('*.cu'))


def _deps_hash(src: Path) -> str:
    h = hashlib.sha1()
    h.update(' '.join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.rglob('*.cuh')) + sorted(CSRC.rglob('*.h')):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, verbose: bool) -> Path:
    rel = src.relative_to(CSRC)
    obj = OBJ_DIR / rel.with_suffix('.o')
    stamp = obj.with_suffix('.sha1')
    digest = _deps_hash(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj
    obj.parent.mkdir(parents=True, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, '-I', str(CSRC), '-c', str(src), '-o', str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = obj.with_suffix('.log')
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f'nvcc failed for {src}:\n{res.stdout}\n{res.stderr}')
    if verbose:
        sys.stderr.write(f'[build_ext] compiled {rel}\n')
    stamp.write_text(digest)
    return obj


def build(verbose: bool = True, force: bool = False) -> Path:
    """Compile every ``.cu`` under ``csrc/`` and link ``lib/libmcb200.so``. Returns the library path."""
    if force and OBJ_DIR.exists():
        shutil.rmtree(OBJ_DIR)
    srcs = sources()
    if not srcs:
        raise RuntimeError(f'no CUDA sources under {CSRC}')
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose), srcs))
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    out = LIB_DIR / LIB_NAME
    newest = max(o.stat().st_mtime for o in objs)
    if out.exists() and out.stat().st_mtime >= newest and not force:
        return out
    # link next to the target and rename: a process (or a copy of the tree) never sees a half-written library
    tmp = out.with_name(out.name + f'.tmp{os.getpid()}')
    cmd = [_nvcc(), '-shared', '-o', str(tmp), *map(str, objs), '-gencode', 'arch=compute_100a,code=sm_100a']
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f'link failed:\n{res.stdout}\n{res.stderr}')
    os.replace(tmp, out)
    if verbose:
        sys.stderr.write(f'[build_ext] linked {out}\n')
    return out


if __name__ == '__main__':
    build(force='--force' in sys.argv)
