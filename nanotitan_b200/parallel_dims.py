"""DP x PP x EP rank layout and the four process-group families.

Rank formula (reference: src/parallel_dims.py:26-31): expert-parallel is the
innermost axis, pipeline the middle, data-parallel the outermost::

    global_rank = (dp * pp_size + pp) * ep_size + ep

Data is sharded over dp*ep ("DP folded over EP"): every EP rank reads its own shard.
`RankLayout` is pure arithmetic (unit-testable with no process group); `ParallelDims`
adds the groups.  All ranks create all groups in the same order, as
`torch.distributed.new_group` requires.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch.distributed as dist

from nanotitan_b200.config import RuntimeConfig
from nanotitan_b200.dist_env import get_local_rank, get_rank, get_world_size, is_distributed


@dataclass
class RankLayout:
    world_size: int
    global_rank: int
    dp_size: int
    pp_size: int
    ep_size: int
    num_experts: int = 1
    dp_rank: int = field(init=False)
    pp_rank: int = field(init=False)
    ep_rank: int = field(init=False)

    def __post_init__(self) -> None:
        assert self.pp_size * self.dp_size * self.ep_size == self.world_size, (
            f"dp({self.dp_size})*pp({self.pp_size})*ep({self.ep_size}) != world({self.world_size})"
        )
        assert self.num_experts % self.ep_size == 0, (
            "Number of experts should be divisible by the size of expert group"
        )
        self.dp_rank = self.global_rank // (self.pp_size * self.ep_size)
        self.pp_rank = (self.global_rank // self.ep_size) % self.pp_size
        self.ep_rank = self.global_rank % self.ep_size

    # -- coordinates ---------------------------------------------------------------
    def rank_of(self, dp: int, pp: int, ep: int) -> int:
        return (dp * self.pp_size + pp) * self.ep_size + ep

    @property
    def data_world_size(self) -> int:
        return self.dp_size * self.ep_size

    @property
    def data_rank(self) -> int:
        return self.dp_rank * self.ep_size + self.ep_rank

    @property
    def is_pp_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_pp_last_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    @property
    def prev_pp_rank(self) -> int:
        return -1 if self.is_pp_first_stage else self.global_rank - self.ep_size

    @property
    def next_pp_rank(self) -> int:
        return -1 if self.is_pp_last_stage else self.global_rank + self.ep_size

    # -- group membership tables (every family partitions the world) ---------------
    def all_ep_groups(self) -> list[list[int]]:
        return [
            [self.rank_of(dp, pp, ep) for ep in range(self.ep_size)]
            for dp in range(self.dp_size)
            for pp in range(self.pp_size)
        ]

    def all_pp_groups(self) -> list[list[int]]:
        return [
            [self.rank_of(dp, pp, ep) for pp in range(self.pp_size)]
            for dp in range(self.dp_size)
            for ep in range(self.ep_size)
        ]

    def all_shared_dp_groups(self) -> list[list[int]]:
        """Replicas of the non-expert parameters of one stage: dp*ep ranks."""
        return [
            [self.rank_of(dp, pp, ep) for dp in range(self.dp_size) for ep in range(self.ep_size)]
            for pp in range(self.pp_size)
        ]

    def all_expert_dp_groups(self) -> list[list[int]]:
        """Replicas of one expert shard of one stage: dp ranks."""
        return [
            [self.rank_of(dp, pp, ep) for dp in range(self.dp_size)]
            for pp in range(self.pp_size)
            for ep in range(self.ep_size)
        ]

    @staticmethod
    def _mine(groups: list[list[int]], rank: int) -> list[int]:
        return next(g for g in groups if rank in g)

    @property
    def ep_group_ranks(self) -> list[int]:
        return self._mine(self.all_ep_groups(), self.global_rank)

    @property
    def pp_group_ranks(self) -> list[int]:
        return self._mine(self.all_pp_groups(), self.global_rank)

    @property
    def shared_dp_group_ranks(self) -> list[int]:
        return self._mine(self.all_shared_dp_groups(), self.global_rank)

    @property
    def expert_dp_group_ranks(self) -> list[int]:
        return self._mine(self.all_expert_dp_groups(), self.global_rank)


class ParallelDims(RankLayout):
    """`RankLayout` of this process plus its ep / pp / shared-dp / expert-dp groups."""

    def __init__(self, config: RuntimeConfig, build_groups: bool = True):
        RankLayout.__init__(
            self,
            world_size=get_world_size(),
            global_rank=get_rank(),
            dp_size=config.dp_size,
            pp_size=config.pp_size,
            ep_size=config.ep_size,
            num_experts=config.num_expert,
        )
        self.local_rank = get_local_rank()
        self.ep_group = self.pp_group = self.shared_dp_group = self.expert_dp_group = None
        if build_groups and is_distributed():
            self.ep_group = self._build(self.all_ep_groups())
            self.pp_group = self._build(self.all_pp_groups())
            self.shared_dp_group = self._build(self.all_shared_dp_groups())
            self.expert_dp_group = self._build(self.all_expert_dp_groups())

    def _build(self, families: list[list[int]]):
        mine = None
        for ranks in families:
            group = dist.new_group(ranks=ranks)
            if self.global_rank in ranks:
                mine = group
        return mine

    def __repr__(self) -> str:
        return (
            f"ParallelDims(rank={self.global_rank} dp={self.dp_rank}/{self.dp_size} "
            f"pp={self.pp_rank}/{self.pp_size} ep={self.ep_rank}/{self.ep_size} "
            f"ep_group={self.ep_group_ranks} pp_group={self.pp_group_ranks} "
            f"shared_dp={self.shared_dp_group_ranks} expert_dp={self.expert_dp_group_ranks})"
        )


def get_parallel_dims(config: RuntimeConfig) -> ParallelDims:
    return ParallelDims(config)
