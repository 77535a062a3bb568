"""Collective-order checker on gloo ranks: matching sequences pass, a different operation or size raises on every rank
before anything is launched, a rank that never arrives ends the others' wait with an error instead of a hang."""
import torch

from dist_utils import run_ranks


def _worker(rank, world, case):
    import torch.distributed as dist

    from mcore_bridge_b200.parallel.collective_check import (CollectiveMismatch, CollectiveOrderChecker,
                                                             CollectiveTimeout)
    orig = dist.all_reduce
    out = 'ok'
    with CollectiveOrderChecker(timeout_s=3.0):
        assert dist.all_reduce is not orig
        t = torch.ones(8)
        dist.all_reduce(t)                                   # collective #0: the same everywhere
        assert t[0].item() == world
        sub = dist.new_group(list(range(world)))             # same members: one sequence with the default group
        dist.broadcast(t, src=0, group=sub)
        try:
            if case == 'match':
                dist.all_reduce(torch.ones(4))
                dist.barrier()
            elif case == 'op':
                if rank == 1:
                    dist.broadcast(torch.ones(4), src=0)
                else:
                    dist.all_reduce(torch.ones(4))
            elif case == 'size':
                dist.all_reduce(torch.ones(4 + rank))
            elif case == 'missing':
                if rank != 1:
                    dist.all_reduce(torch.ones(4))
        except CollectiveMismatch as e:
            out = 'mismatch: ' + str(e)
        except CollectiveTimeout as e:
            out = 'timeout: ' + str(e)
    assert dist.all_reduce is orig                           # removed on exit
    return out


def test_matching_sequences_pass():
    assert run_ranks(_worker, 2, 'match') == ['ok', 'ok']


def test_different_operation_raises_on_both_ranks():
    res = run_ranks(_worker, 2, 'op')
    assert all(r.startswith('mismatch') for r in res), res
    assert 'all_reduce(4xfloat32)' in res[0] and 'broadcast(4xfloat32)' in res[0] and 'collective #2' in res[0]


def test_different_size_raises():
    res = run_ranks(_worker, 2, 'size')
    assert all(r.startswith('mismatch') for r in res), res
    assert '4xfloat32' in res[1] and '5xfloat32' in res[1]


def test_missing_rank_ends_the_wait_with_an_error():
    res = run_ranks(_worker, 3, 'missing')
    assert res[1] == 'ok' and res[0].startswith('timeout') and res[2].startswith('timeout')
    assert 'rank 1 did not reach collective #2' in res[0]
