"""MoE layer as a composition of PyTorch ops plus NCCL/gloo all-to-all.

Same math and data flow as the reference's torch backend
(src/model/torch_backend.py:24-157): fp32 router -> softmax -> top-k -> renormalise,
expert-major packing in ascending token order, count exchange + row all-to-all +
regroup by local expert when ep_size > 1, experts, the reverse path, gate-weighted
scatter-add.  Every Python loop of the reference is replaced by a vectorised index
computation, so the only host syncs are the split sizes the collective needs.  This
is the CPU path and the unfused baseline the fused EP kernels are measured against.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from nanotitan_b200.models.utils import ModelShardSpec, MoELayerStats
from nanotitan_b200.ops import moe as moe_ops
from nanotitan_b200.ops import reference as ref
from nanotitan_b200.profiler import nvtx_range


class TorchMoEBackend:
    def __init__(self, cfg, experts: nn.Module, router: nn.Linear, spec: ModelShardSpec):
        self.cfg, self.spec, self.router, self.experts = cfg, spec, router, experts
        # False: the load-balancing loss back-propagates into the tokens (the reference's torch
        # backend).  True: it sees detached tokens, as the CUDA backends do.
        self.aux_on_detached_tokens = False

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        batch, seq_len, d_model = x.shape
        flat = x.reshape(-1, d_model)
        num_experts = self.cfg.num_experts

        with nvtx_range("moe/router"):
            gates, top_e, probs = ref.router_topk(flat, self.router.weight, self.cfg.top_k)
        assert gates.dtype == torch.float32, "Expert topk weights should be in fp32"

        with nvtx_range("moe/pack_tokens"):
            packed_x, packed_token, _, packed_gate, counts = ref.pack_tokens(
                flat, gates, top_e, num_experts
            )

        if self.spec.ep_size == 1:
            expert_in, local_offsets, regroup = packed_x, ref.offsets_from_counts(counts), None
        else:
            ep, group = self.spec.ep_size, self.spec.ep_group
            recv_matrix = moe_ops.exchange_counts(counts, ep, group)  # [src, local expert]
            send_splits = counts.view(ep, -1).sum(dim=1).tolist()
            recv_splits = recv_matrix.sum(dim=1).tolist()
            received = moe_ops.all_to_all_rows(packed_x, send_splits, recv_splits, group)
            regroup = moe_ops.source_major_to_expert_major(recv_matrix)
            expert_in = received[regroup]
            local_offsets = ref.offsets_from_counts(recv_matrix.sum(dim=0))

        with nvtx_range("moe/expert_compute"):
            expert_out = self.experts(expert_in, local_offsets)

        if regroup is not None:
            by_source = torch.empty_like(expert_out)
            by_source[regroup] = expert_out
            expert_out = moe_ops.all_to_all_rows(by_source, recv_splits, send_splits, group)

        with nvtx_range("moe/combine_tokens"):
            out = ref.combine_tokens(expert_out, packed_token, packed_gate, flat.shape[0], flat.dtype)
        if residual is not None:
            out = out + residual.reshape(-1, d_model)

        if self.aux_on_detached_tokens:
            probs = ref.router_topk(flat.detach(), self.router.weight, self.cfg.top_k)[2]
        stats = MoELayerStats(counts.detach(), probs_per_expert=probs, cfg=self.cfg)
        return out.reshape(batch, seq_len, d_model), stats
