"""Host-side logic of the expert-parallel exchange that needs no GPU: the pool of symmetric buffers
(every rank must pick the same buffer for the same role, step after step) and the capacity rule.
The exchange object is built without its constructor (no symmetric memory on a CPU box) and given an
allocator that hands out numbered fake buffers."""
import torch

from nanotitan_b200.parallel.ep_fused import FusedExchange, _SymmBuffer


def _exchange(ep=4, factor=0.0):
    ex = object.__new__(FusedExchange)
    ex.ep, ex.capacity_factor = ep, factor
    ex._free, ex._used, ex._fixed, ex.allocated_bytes = [], [], {}, 0
    return ex


class _Tagged(_SymmBuffer):
    """A fake symmetric buffer; `tag` = allocation order = identity of the allocation across ranks."""

    __slots__ = ("tag",)


def _run_steps(ex, layers, steps, capacity, assignments, d=8):
    """The acquire / release order of `steps` training steps of a model with `layers` MoE layers."""
    picks = []
    for _ in range(steps):
        ex.reset()
        held = []
        for _ in range(layers):  # forward: two buffers per layer
            x_in = ex.acquire(capacity, d, torch.bfloat16)
            y_home = ex.acquire(assignments, d, torch.bfloat16)
            held.append((x_in, y_home))
            picks.append((id(x_in), id(y_home)))
        for x_in, y_home in reversed(held):  # backward: the return transfer's node runs first
            ex.release(y_home)
            ex.release(x_in)
    return picks


def _fresh(ep=4):
    ex = _exchange(ep)
    made = []

    def new_buffer(numel, dtype):
        buf = _Tagged(torch.empty(numel, dtype=dtype), torch.zeros(ep, dtype=torch.int64))
        buf.tag = len(made)
        made.append(buf)
        return buf

    ex._new_buffer = new_buffer
    return ex, made


def test_two_ranks_walk_their_pools_identically():
    a, made_a = _fresh()
    b, made_b = _fresh()
    for ex in (a, b):
        _run_steps(ex, layers=5, steps=3, capacity=64, assignments=16)
    assert len(made_a) == len(made_b) == 10  # two per layer, allocated in the first step only
    assert [buf.tag for buf in a._free] == [buf.tag for buf in b._free]


def test_steady_state_reuses_buffers_without_allocating():
    ex, made = _fresh()
    _run_steps(ex, layers=4, steps=1, capacity=64, assignments=16)
    before = len(made)
    picks = _run_steps(ex, layers=4, steps=4, capacity=64, assignments=16)
    assert len(made) == before
    per_step = [picks[i * 4:(i + 1) * 4] for i in range(4)]
    # backward releases in reverse layer order, so layer l inherits the buffers layer L-1-l used in the
    # step before: the assignment has period two (a captured step bakes one of the two in)
    assert per_step[0] == per_step[2] and per_step[1] == per_step[3]
    assert sorted(per_step[0]) == sorted(per_step[1])
    for x_in, y_home in picks:
        assert x_in != y_home


def test_a_request_never_gets_a_buffer_that_is_too_small():
    ex, _ = _fresh()
    small = ex.acquire(4, 8, torch.bfloat16)
    ex.release(small)
    big = ex.acquire(400, 8, torch.bfloat16)
    assert big is not small and big.numel >= 3200
    ex.release(big)
    assert ex.acquire(4, 8, torch.bfloat16) is small  # first fit in pool order


def test_reset_returns_buffers_whose_backward_never_ran():
    ex, made = _fresh()
    ex.acquire(64, 8, torch.bfloat16)
    ex.acquire(16, 8, torch.bfloat16)
    assert len(ex._used) == 2
    ex.reset()
    assert not ex._used and len(ex._free) == 2
    ex.acquire(64, 8, torch.bfloat16)
    assert len(made) == 2


def test_fixed_buffers_are_allocated_once_and_grow_on_demand():
    ex, made = _fresh()
    a = ex.fixed("dx_home", 16, 8, torch.bfloat16)
    assert ex.fixed("dx_home", 16, 8, torch.bfloat16) is a
    b = ex.fixed("dx_home", 32, 8, torch.bfloat16)
    assert b is not a and len(made) == 2


def test_capacity_is_the_worst_case_unless_bounded():
    assert _exchange(ep=4).capacity_rows(1000) == 4000
    assert _exchange(ep=8).capacity_rows(24576) == 8 * 24576
    bounded = _exchange(ep=8, factor=2.0)
    assert bounded.capacity_rows(24576) == 49152
    assert bounded.capacity_rows(100) == 256            # rounded up to whole 128-row tiles
    assert _exchange(ep=2, factor=4.0).capacity_rows(1000) == 2000  # never above the worst case
    assert _exchange(ep=4).capacity_rows(0) == 128
