"""A host model of the expert-parallel exchange's row layout (csrc/kernels/ep_exchange.cu), for layouts no
single-GPU test reaches: 8 ranks, collapsed routing, empty experts.

The model restates the three segment tables the kernels build from the all-gathered count matrix
`cmat[source rank, expert]` and checks what the exchange relies on:
  * dispatch writes every (source rank, packed row) to exactly one staging row of the expert's rank, the rows of
    one expert are contiguous there and ordered by source rank, and nothing lands past the rows that rank expects;
  * the return transfer (direction 1) sends every staging row back to the packed row it came from;
  * the backward of the return (direction 0) addresses the same staging rows as dispatch did;
  * the rank-rotated walk of `ep_push_rows` visits every row once.
"""
import numpy as np
import pytest


def _routing(rng, tokens, k, experts, skew):
    """Top-k expert ids per token; `skew` > 0 sends most tokens to the first two experts, as a freshly
    initialised deep router does."""
    logits = rng.standard_normal((tokens, experts))
    logits[:, :2] += skew
    return np.argsort(-logits, axis=1)[:, :k]


def _plan(idx, experts):
    """counts, exclusive offsets and the packed slot of every (token, j): expert-major, token order."""
    flat = idx.reshape(-1)
    counts = np.bincount(flat, minlength=experts)
    order = np.argsort(flat, kind="stable")
    slot = np.empty_like(order)
    slot[order] = np.arange(flat.size)
    return counts, np.concatenate([[0], np.cumsum(counts)]), slot.reshape(idx.shape)


def _last_segment_at_or_before(seg_start, n_segments, r):
    lo, hi = 0, n_segments  # the kernel's search: last segment whose start is <= r (empty segments share a start)
    while hi - lo > 1:
        mid = (lo + hi) >> 1
        if seg_start[mid] <= r:
            lo = mid
        else:
            hi = mid
    return lo


def _push_tables(cmat, me, ep, experts, direction):
    e_loc_n = experts // ep
    start, peer, dst0 = np.zeros(experts + 1, np.int64), np.zeros(experts, np.int64), np.zeros(experts, np.int64)
    for g in range(experts):
        if direction == 0:  # packed rows of this rank, by expert -> staging rows on the expert's rank
            e = g
            peer[g] = e // e_loc_n
            start[g] = cmat[me, :e].sum()
            dst0[g] = cmat[:, peer[g] * e_loc_n : e].sum() + cmat[:me, e].sum()
        else:  # staging rows of this rank, by (local expert, source) -> packed rows on the source
            e_loc, s = divmod(g, ep)
            e = me * e_loc_n + e_loc
            peer[g] = s
            start[g] = cmat[:, me * e_loc_n : e].sum() + cmat[:s, e].sum()
            dst0[g] = cmat[s, :e].sum()
    start[experts] = cmat[me].sum() if direction == 0 else cmat[:, me * e_loc_n : (me + 1) * e_loc_n].sum()
    return start, peer, dst0


@pytest.mark.parametrize("tokens,k,experts,ep,skew", [(96, 2, 8, 8, 0.0), (200, 2, 8, 8, 4.0), (64, 8, 64, 8, 0.0),
                                                     (150, 2, 8, 4, 4.0), (40, 1, 4, 2, 0.0), (33, 2, 16, 8, 6.0)])
def test_every_row_has_one_place_and_comes_back(tokens, k, experts, ep, skew):
    rng = np.random.default_rng(tokens + experts + ep)
    e_loc_n, A = experts // ep, tokens * k
    plans = [_plan(_routing(rng, tokens, k, experts, skew), experts) for _ in range(ep)]
    cmat = np.stack([p[0] for p in plans])
    expected = [int(cmat[:, r * e_loc_n : (r + 1) * e_loc_n].sum()) for r in range(ep)]
    capacity = ep * A  # the default: worst case
    staging = [np.full(capacity, -1, np.int64) for _ in range(ep)]

    # ---- dispatch: destination row = rows of earlier experts of that rank (all sources) + rows of the same expert
    # from earlier sources + position within my rows of the expert
    for me, (counts, offsets, _) in enumerate(plans):
        for e in range(experts):
            peer = e // e_loc_n
            dst0 = cmat[:, peer * e_loc_n : e].sum() + cmat[:me, e].sum() - offsets[e]
            for slot in range(offsets[e], offsets[e + 1]):
                dst = dst0 + slot
                assert 0 <= dst < expected[peer] <= capacity
                assert staging[peer][dst] == -1, "two rows were given the same staging row"
                staging[peer][dst] = me * A + slot
    for r in range(ep):
        assert (staging[r][: expected[r]] >= 0).all() and (staging[r][expected[r] :] == -1).all()
        sources = staging[r][: expected[r]] // A
        bounds = np.concatenate([[0], np.cumsum(cmat[:, r * e_loc_n : (r + 1) * e_loc_n].sum(0))])
        for lo, hi in zip(bounds[:-1], bounds[1:]):  # within one expert: ordered by source rank
            assert (np.diff(sources[lo:hi]) >= 0).all()

    for me in range(ep):
        # ---- return: every staging row goes to the packed row it came from
        start, peer, dst0 = _push_tables(cmat, me, ep, experts, direction=1)
        assert (np.diff(start) >= 0).all() and start[experts] == expected[me]
        for r in range(expected[me]):
            g = _last_segment_at_or_before(start, experts, r)
            assert start[g] <= r < start[g + 1]
            dst = dst0[g] + (r - start[g])
            assert 0 <= dst < A and staging[me][r] == peer[g] * A + dst
        # ---- backward of the return: packed rows find the staging rows dispatch used
        start, peer, dst0 = _push_tables(cmat, me, ep, experts, direction=0)
        assert start[experts] == A
        for r in range(A):
            g = _last_segment_at_or_before(start, experts, r)
            assert staging[peer[g]][dst0[g] + (r - start[g])] == me * A + r
        # ---- the rotated walk: start at the first row bound for rank me + 1, wrap around
        for direction, rows in ((0, A), (1, expected[me])):
            start, _, _ = _push_tables(cmat, me, ep, experts, direction)
            first = (me + 1) % ep
            rot = min(start[first * e_loc_n if direction == 0 else first], rows)
            visited = sorted((r0 + rot) - rows if r0 + rot >= rows else r0 + rot for r0 in range(rows))
            assert visited == list(range(rows))
