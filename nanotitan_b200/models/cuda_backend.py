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
from nanotitan_b200.profiler import nvtx_range


_CONSTANTS: dict = {}


def _single_expert_constants(device, assignments: int, alpha: float):
    """(counts int32 [1], ones fp32 [1], alpha fp32 scalar) for a one-expert layer, made once per device."""
    key = (device, assignments, alpha)
    hit = _CONSTANTS.get(key)
    if hit is None:
        hit = (
            torch.full((1,), assignments, dtype=torch.int32, device=device),
            torch.ones(1, dtype=torch.float32, device=device),
            torch.full((), alpha, dtype=torch.float32, device=device),
        )
        _CONSTANTS[key] = hit
    return hit


class _ZeroGradLink(torch.autograd.Function):
    """Returns the constant `value` while keeping `weight` in the graph with an exactly-zero gradient."""

    @staticmethod
    def forward(ctx, weight, value):
        ctx.weight = weight
        return value.view_as(value)

    @staticmethod
    def backward(ctx, _grad):
        from nanotitan_b200.ops import native

        dw = native.grad_buffer(ctx.weight)
        return dw.zero_(), None


class CUDAMoEBackend:
    # False: the load-balancing loss sees detached tokens (the reference's CUDA backend); True: its
    # gradient also reaches the tokens (the reference's torch backend) - set for loss-parity runs
    # against that backend.
    aux_to_tokens = False

    def __init__(self, cfg, experts: nn.Module, router: nn.Linear, spec: ModelShardSpec | None = None):
        self.cfg, self.router, self.experts = cfg, router, experts
        self.spec = spec if spec is not None else ModelShardSpec.full(cfg)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        batch, seq_len, d_model = x.shape
        flat = x.reshape(-1, d_model)
        if not flat.is_cuda:
            raise RuntimeError(f"moe_backend='cuda' needs GPU tensors (got {flat.device})")
        res = None if residual is None else residual.reshape(-1, d_model)
        if self.cfg.num_experts == 1 and self.spec.ep_size == 1:
            # One expert: routing is the identity (gate 1, every token in place), so the layer is
            # the dense SwiGLU FFN with the residual folded into the down-projection.  The router
            # gets no gradient signal (softmax over one logit), exactly as in the general path.
            from nanotitan_b200.ops import native

            tokens = flat.shape[0]
            offsets = native.whole_segment(tokens, flat.device)
            with nvtx_range("moe/expert_compute"):
                out = native.swiglu_experts(flat, self.experts.W_gate, self.experts.W_val, self.experts.W_out, offsets, res)
            # Routing statistics are constants here (fraction 1, probability 1); the loss is tied to
            # the router weight by a node whose backward is one zero-fill, which is the gradient
            # softmax over a single logit gives.
            counts, ones, alpha = _single_expert_constants(flat.device, tokens * self.cfg.top_k, float(self.cfg.router_alpha))
            aux = _ZeroGradLink.apply(self.router.weight, alpha) if self.router.weight.requires_grad else alpha
            stats = MoELayerStats.single_expert(self.cfg, counts, ones, aux)
            return out.reshape(batch, seq_len, d_model), stats
        elif self.spec.ep_size > 1:
            from nanotitan_b200.parallel.ep import expert_parallel_moe

            out, counts, probs_mean = expert_parallel_moe(self, flat, res)
        else:
            from nanotitan_b200.ops import native

            with nvtx_range("moe/router"):
                gates, top_e, counts, probs_mean = native.router_topk_mean(flat, self.router.weight, self.cfg.top_k, self.aux_to_tokens)
            with nvtx_range("moe/pack_tokens"):
                packed_x, packed_gate, packed_token, _, offsets, slot_of = native.pack(flat, gates, top_e, counts)
            with nvtx_range("moe/expert_compute"):
                expert_out = self.experts(packed_x, offsets)
            with nvtx_range("moe/combine_tokens"):
                out = native.combine(expert_out, packed_gate, packed_token, slot_of, flat.shape[0], res)
        stats = MoELayerStats(counts.detach(), probs_per_expert=probs_mean, cfg=self.cfg,
                              assignments=flat.shape[0] * self.cfg.top_k)
        return out.reshape(batch, seq_len, d_model), stats
