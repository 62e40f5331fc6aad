"""Model sharding spec (which layers / experts a rank owns) and per-layer MoE statistics.

Reference: src/model/utils.py:10-93.  Layers are split into contiguous blocks of
n_layers/pp_size per pipeline stage, embeddings live on the first stage, the unembed
head on the last, and experts are split contiguously over the expert-parallel ranks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch


@dataclass(frozen=True)
class ModelShardSpec:
    layer_start: int
    layer_end: int
    has_token_embed: bool
    has_pos_embed: bool
    has_unembed_head: bool
    per_rank_expert: int
    start_expert_id: int
    end_expert_id: int
    ep_size: int = 1
    ep_group: Any = None

    @classmethod
    def full(cls, cfg) -> "ModelShardSpec":
        """The whole model on one rank."""
        return cls(0, cfg.n_layers, True, True, True, cfg.num_experts, 0, cfg.num_experts)


def get_layer_bounds(cfg, pp_rank: int) -> tuple[int, int]:
    per_stage = cfg.model.n_layers // cfg.runtime.pp_size
    return pp_rank * per_stage, (pp_rank + 1) * per_stage


def get_logical_expert_bounds(ep_rank: int, num_per_rank_experts: int) -> tuple[int, int]:
    lo = ep_rank * num_per_rank_experts
    return lo, lo + num_per_rank_experts


def get_model_shard_specs(dim, cfg) -> ModelShardSpec:
    layer_start, layer_end = get_layer_bounds(cfg, dim.pp_rank)
    per_rank = dim.num_experts // dim.ep_size
    lo, hi = get_logical_expert_bounds(dim.ep_rank, per_rank)
    return ModelShardSpec(
        layer_start=layer_start,
        layer_end=layer_end,
        has_token_embed=dim.is_pp_first_stage,
        has_pos_embed=dim.is_pp_first_stage,
        has_unembed_head=dim.is_pp_last_stage,
        per_rank_expert=per_rank,
        start_expert_id=lo,
        end_expert_id=hi,
        ep_size=dim.ep_size,
        ep_group=dim.ep_group,
    )


@dataclass
class MoELayerStats:
    """Routing statistics of one layer and its Switch-style load-balancing loss.

    aux = alpha * E * sum_e frac_e * P_e with frac_e the fraction of assignments
    routed to expert e and P_e the mean router probability of expert e
    (reference: src/model/utils.py:70-93).  `probs_per_expert` may be the [T, E]
    probabilities or their mean over tokens [E].
    """

    tokens_per_expert: torch.Tensor
    probs_per_expert: torch.Tensor
    cfg: Any
    aux_loss: torch.Tensor | None = None
    # number of (token, choice) assignments when the caller knows it on the host (tokens * top_k):
    # the fractions are then a multiplication by a constant and the loss a single dot product
    assignments: int | None = None

    @classmethod
    def single_expert(cls, cfg, tokens_per_expert, ones, aux_loss):
        """Statistics of a layer with one expert, where every quantity is known without arithmetic:
        fraction 1, mean probability 1, loss alpha * 1 * (1 * 1).  The caller passes cached
        constants (`ones` is a float [1] tensor of 1.0), so no kernel runs."""
        stats = object.__new__(cls)
        stats.tokens_per_expert = tokens_per_expert
        stats.probs_per_expert = ones
        stats.cfg = cfg
        stats.num_tokens = None
        stats.assignments = None
        stats._total = tokens_per_expert.sum() if tokens_per_expert.numel() != 1 else tokens_per_expert[0]
        stats._frac = ones
        stats.aux_loss = aux_loss
        return stats

    def __post_init__(self) -> None:
        if self.probs_per_expert.ndim == 2:
            self.num_tokens = self.probs_per_expert.shape[0]
            self.probs_per_expert = self.probs_per_expert.mean(dim=0)
        else:
            self.num_tokens = None
        assert self.tokens_per_expert.shape == self.probs_per_expert.shape
        assert self.tokens_per_expert.ndim == 1
        self._total = self._frac = None
        scale = self.cfg.router_alpha * self.cfg.num_experts
        if self.assignments:
            self.aux_loss = torch.dot(self.tokens_per_expert.float(), self.probs_per_expert.float()) * (scale / self.assignments)
        else:
            self.aux_loss = scale * torch.sum(self.ass_frac_per_expert * self.probs_per_expert.float())

    @property
    def total_assignments(self) -> torch.Tensor:
        if self._total is None:
            self._total = self.tokens_per_expert.sum()
        return self._total

    @property
    def ass_frac_per_expert(self) -> torch.Tensor:
        if self._frac is None:
            self._frac = self.tokens_per_expert.float() / self.total_assignments
        return self._frac
