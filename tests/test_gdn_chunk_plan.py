"""Chunked gated delta rule over packed batches: sequences of unequal length in any order, an empty sequence, tokens
outside every sequence, lengths that are and are not whole chunks — against the token-by-token definition, values and
gradients; and the host-side copy of the sequence boundaries."""
import pytest
import torch


def _inputs(T, h=3, dk=16, dv=24, seed=0):
    from mcore_bridge_b200.ops import gdn as G
    g = torch.Generator().manual_seed(seed)
    q, k = G.l2norm(torch.randn(T, h, dk, generator=g)), G.l2norm(torch.randn(T, h, dk, generator=g))
    v = torch.randn(T, h, dv, generator=g)
    decay = -torch.rand(T, h, generator=g) * 0.5
    beta = torch.rand(T, h, generator=g)
    return q, k, v, decay, beta


@pytest.mark.parametrize('T,cu', [(333, None), (333, [0, 70, 70, 200, 333]), (333, [5, 100, 229]),
                                  (256, [0, 64, 128, 256]), (300, [0, 17, 211, 300])])
def test_chunked_rule_equals_the_recurrence(T, cu):
    from mcore_bridge_b200.ops import gdn as G
    cut = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    a_in = [x.clone().requires_grad_() for x in _inputs(T)]
    b_in = [x.clone().requires_grad_() for x in _inputs(T)]
    a = G.chunk_gated_delta_rule(*a_in, cut)
    b = G.recurrent_gated_delta_rule(*b_in, cut)
    assert (a - b).abs().max().item() < 2e-6
    if cu is not None:                                   # tokens outside every sequence produce zeros
        outside = torch.ones(T, dtype=torch.bool)
        for s, e in zip(cu[:-1], cu[1:]):
            outside[s:e] = False
        assert a[outside].abs().sum().item() == 0
    go = torch.randn(a.shape, generator=torch.Generator().manual_seed(1))
    a.backward(go)
    b.backward(go)
    for x, y in zip(a_in, b_in):
        assert (x.grad - y.grad).abs().max().item() < 2e-5


def test_plan_is_shared_between_calls_and_sorted_by_length():
    from mcore_bridge_b200.ops import gdn as G
    G._chunk_plan.cache_clear()
    bounds = ((0, 17), (17, 211), (211, 300))
    p = G._chunk_plan(bounds, 300, 64, 'cpu')
    assert p.alive == (3, 2, 1, 1) and p.n_seq == 3 and p.total == 1 + 4 + 2 and not p.identity
    assert p.first.tolist() == [0, 4, 6]                 # longest sequence first
    assert G._chunk_plan(bounds, 300, 64, 'cpu') is p and G._chunk_plan.cache_info().hits == 1
    assert G._chunk_plan(((0, 128),), 128, 64, 'cpu').identity


def test_boundaries_are_read_from_the_host_copy():
    from mcore_bridge_b200.utils.torch_utils import attach_host_list, host_list
    host = torch.tensor([0, 5, 9], dtype=torch.int32)
    dev = host.clone()
    assert host_list(dev) == [0, 5, 9]
    attach_host_list(dev, host)
    dev.zero_()                                           # the attached values are what is read, not the tensor
    assert host_list(dev) == [0, 5, 9]
