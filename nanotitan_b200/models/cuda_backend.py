"""MoE layer on the fused sm_100a kernels.

Data flow of the reference's CUDA backend (src/model/cuda_backend.py:18-81) —
router, top-k, count, pack, experts, combine — with these differences: the router,
softmax, top-k, renormalisation and per-expert counting are one kernel; slots come
from a deterministic scan (ascending token id within an expert) instead of atomics;
the three expert GEMMs are tcgen05 grouped GEMMs with the SwiGLU folded into the
up-projection epilogue; combine is an atomic-free gather that also adds the residual;
and expert parallelism is supported (the reference's CUDA backend is single-rank).
The load-balancing loss sees router probabilities computed from *detached* tokens, as
in the reference (src/model/cuda_backend.py:39-41): its gradient reaches the router
weight only.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from nanotitan_b200.models.utils import ModelShardSpec, MoELayerStats
from nanotitan_b200.ops import moe as moe_ops
from nanotitan_b200.profiler import nvtx_range


class CUDAMoEBackend:
    def __init__(self, cfg, experts: nn.Module, router: nn.Linear, spec: ModelShardSpec | None = None):
        self.cfg, self.router, self.experts = cfg, router, experts
        self.spec = spec if spec is not None else ModelShardSpec.full(cfg)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        batch, seq_len, d_model = x.shape
        flat = x.reshape(-1, d_model)
        res = None if residual is None else residual.reshape(-1, d_model)
        if self.spec.ep_size > 1:
            from nanotitan_b200.parallel.ep import expert_parallel_moe

            out, counts, probs_mean = expert_parallel_moe(self, flat, res)
        else:
            with nvtx_range("moe/router"):
                gates, top_e, probs_mean, counts = moe_ops.router_topk(
                    flat, self.router.weight, self.cfg.top_k, native=True
                )
            with nvtx_range("moe/pack_tokens"):
                packed_x, packed_token, _, packed_gate, counts = moe_ops.pack_tokens(
                    flat, gates, top_e, self.cfg.num_experts, native=True
                )
                offsets = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=x.device)
                offsets[1:] = torch.cumsum(counts, dim=0)
            with nvtx_range("moe/expert_compute"):
                expert_out = self.experts(packed_x, offsets)
            with nvtx_range("moe/combine_tokens"):
                out = moe_ops.combine_tokens(
                    expert_out, packed_token, packed_gate, flat.shape[0], res, native=True
                )
        stats = MoELayerStats(counts.detach(), probs_per_expert=probs_mean, cfg=self.cfg)
        return out.reshape(batch, seq_len, d_model), stats
