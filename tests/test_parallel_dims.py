"""Rank layout arithmetic: no process group needed."""
import itertools

import pytest

from nanotitan_b200.parallel_dims import RankLayout


@pytest.mark.parametrize("dp,pp,ep", [(1, 1, 1), (2, 1, 1), (2, 2, 1), (1, 2, 4), (2, 2, 2), (1, 1, 8)])
def test_families_partition_the_world(dp, pp, ep):
    world = dp * pp * ep
    lay = RankLayout(world, 0, dp, pp, ep, num_experts=8)
    for fam, size in ((lay.all_ep_groups(), ep), (lay.all_pp_groups(), pp),
                      (lay.all_shared_dp_groups(), dp * ep), (lay.all_expert_dp_groups(), dp)):
        assert all(len(g) == size for g in fam)
        assert sorted(itertools.chain.from_iterable(fam)) == list(range(world))


def test_rank_formula_ep_innermost_pp_middle_dp_outermost():
    lay = RankLayout(8, 5, dp_size=1, pp_size=2, ep_size=4, num_experts=16)
    assert (lay.dp_rank, lay.pp_rank, lay.ep_rank) == (0, 1, 1)
    assert lay.ep_group_ranks == [4, 5, 6, 7]
    assert lay.pp_group_ranks == [1, 5]
    assert lay.shared_dp_group_ranks == [4, 5, 6, 7]
    assert lay.expert_dp_group_ranks == [5]
    assert lay.prev_pp_rank == 1 and lay.next_pp_rank == -1
    assert lay.data_world_size == 4 and lay.data_rank == 1
    assert lay.is_pp_last_stage and not lay.is_pp_first_stage


def test_dp_folded_over_ep_gives_distinct_data_ranks():
    seen = set()
    for r in range(8):
        lay = RankLayout(8, r, dp_size=2, pp_size=1, ep_size=4, num_experts=4)
        seen.add(lay.data_rank)
    assert seen == set(range(8))


def test_invalid_layouts_rejected():
    with pytest.raises(AssertionError):
        RankLayout(8, 0, 2, 2, 1)
    with pytest.raises(AssertionError):
        RankLayout(2, 0, 1, 1, 2, num_experts=3)
