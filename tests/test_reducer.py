"""Bucketed reducer: layout rules on one process, gradient equality on gloo ranks."""
import copy

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from nanotitan_b200.parallel.reducer import ReducerV1, plan_buckets
from tests.conftest import run_distributed


def _params(sizes, dtype=torch.float32):
    return [nn.Parameter(torch.zeros(n, dtype=dtype)) for n in sizes]


def test_buckets_fill_in_reverse_order_and_respect_the_cap():
    params = _params([100, 200, 300, 50])
    buckets = plan_buckets(params, bucket_bytes=1400)  # 350 floats
    assert [[p.numel() for p in b.params] for b in buckets] == [[50, 300], [200, 100]]
    for b in buckets:
        assert b.size_bytes <= 1400
        for (lo, hi), p in zip(b.spans, b.params):
            assert hi - lo == p.numel() and lo % 4 == 0  # 16-byte aligned spans


def test_one_bucket_per_dtype():
    params = _params([8, 8]) + _params([8], torch.bfloat16)
    buckets = plan_buckets(params, 1 << 20)
    assert sorted(str(b.dtype) for b in buckets) == ["torch.bfloat16", "torch.float32"]


def test_grads_are_views_and_missing_grads_are_zero():
    a, b = _params([4, 4])
    red = ReducerV1([a, b], group_size=1, process_group=None, bucket_size=1)
    assert a.grad.data_ptr() == red.grad_view(a).data_ptr()
    red.backward_grad_sync = True
    (a * 2).sum().backward()  # b is never used
    red.prepare_missing_grad()
    red.finalize_backward()
    assert torch.equal(a.grad, torch.full((4,), 2.0)) and torch.equal(b.grad, torch.zeros(4))
    # an outside zero_grad(set_to_none=True) is repaired
    a.grad = None
    red.zero_grad()
    assert a.grad is not None and a.grad.data_ptr() == red.grad_view(a).data_ptr()


def test_accumulates_over_microbatches_and_syncs_once():
    (a,) = _params([3])
    red = ReducerV1([a], 1, None, 1)
    red.zero_grad()
    red.backward_grad_sync = False
    (a * 1.0).sum().backward()
    assert not red.buckets[0].launched
    red.backward_grad_sync = True
    (a * 2.0).sum().backward()
    assert red.buckets[0].launched
    red.finalize_backward()
    assert torch.equal(a.grad, torch.full((3,), 3.0))


def _ddp_worker(rank, world):
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3))
    ref = copy.deepcopy(net)
    red = ReducerV1(list(net.parameters()), world, dist.group.WORLD, bucket_size=1)
    g = torch.Generator().manual_seed(100)
    data = torch.randn(world * 4, 6, generator=g)
    # every rank takes its slice; the reference sees everything
    red.zero_grad()
    red.backward_grad_sync = True
    net(data[rank * 4 : (rank + 1) * 4]).pow(2).mean().backward()
    red.prepare_missing_grad()
    red.finalize_backward()
    ref(data).pow(2).mean().backward()
    for p, q in zip(net.parameters(), ref.parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-5, atol=1e-6)


@pytest.mark.distributed
def test_two_rank_mean_gradient_equals_full_batch_gradient():
    run_distributed(_ddp_worker, 2)
