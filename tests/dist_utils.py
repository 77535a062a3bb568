"""Helpers to run a function on several gloo ranks (CPU) as child processes."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, ret):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        dist.init_process_group('gloo', rank=rank, world_size=world)
        ret[rank] = ('ok', fn(rank, world, *args))
    except Exception:
        ret[rank] = ('err', traceback.format_exc())
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int, *args, timeout: float = 240.0):
    """Runs ``fn(rank, world, *args)`` on ``world`` gloo ranks; returns the list of return values."""
    ctx = mp.get_context('spawn')
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    for p in procs:
        if p.is_alive():
            p.kill()
            raise TimeoutError('a rank did not finish')
    out = []
    for r in range(world):
        status, val = ret.get(r, ('err', 'no result'))
        if status != 'ok':
            raise RuntimeError(f'rank {r} failed:\n{val}')
        out.append(val)
    return out
