"""Expert parallelism for the CUDA MoE backend.

Tokens are routed on their home rank, travel to the rank that owns their expert, run
through the grouped SwiGLU GEMMs there and travel back to be combined.  Experts are
sharded contiguously (`E_loc = E / ep_size` per rank), so expert-major packing on the
home rank is also destination-major.

Two transports move the rows:
  * `exchange = "nccl"`: count exchange + `all_to_all_single` with host-side split sizes +
    a regroup gather (the data flow of the reference's torch backend,
    src/model/torch_backend.py:72-147, with every other step on the native kernels).
  * `exchange = "p2p"` (the default on GPUs): `nanotitan_b200.parallel.ep_fused` - one kernel
    exchanges the counts and stores every token row straight into its expert rank's expert-major
    staging buffer over NVLink, the grouped GEMMs read that buffer in place, one kernel stores
    the expert outputs into the home rank's packed-order buffer and the combine gathers from it
    (no host sync, no packed copy, no regroup pass).
"""
from __future__ import annotations

import torch

from nanotitan_b200.ops import moe as moe_ops
from nanotitan_b200.ops import native
from nanotitan_b200.profiler import nvtx_range


def _nccl_exchange(backend, packed_x, counts):
    """-> (expert_in [R, d] expert-major, local_offsets [E_loc+1] int32, context for the way back)."""
    spec = backend.spec
    ep, group = spec.ep_size, spec.ep_group
    recv_matrix = moe_ops.exchange_counts(counts, ep, group)  # [src, local expert]
    host = torch.stack([counts.view(ep, -1).sum(dim=1), recv_matrix.sum(dim=1)]).tolist()  # the one host sync
    send_splits, recv_splits = host[0], host[1]
    received = moe_ops.all_to_all_rows(packed_x, send_splits, recv_splits, group)
    regroup = moe_ops.source_major_to_expert_major(recv_matrix)
    expert_in = received[regroup]
    local_offsets = torch.zeros(recv_matrix.shape[1] + 1, dtype=torch.int32, device=packed_x.device)
    local_offsets[1:] = torch.cumsum(recv_matrix.sum(dim=0), dim=0)
    return expert_in, local_offsets, (regroup, send_splits, recv_splits, group)


def _nccl_return(expert_out, ctx):
    regroup, send_splits, recv_splits, group = ctx
    by_source = torch.empty_like(expert_out)
    by_source[regroup] = expert_out
    return moe_ops.all_to_all_rows(by_source, recv_splits, send_splits, group)


def expert_parallel_moe(backend, flat: torch.Tensor, residual: torch.Tensor | None):
    """Forward of one expert-parallel MoE layer on GPU tensors.

    Returns (out [T, d], counts [E] of this rank's routing, mean router probabilities [E])."""
    cfg = backend.cfg
    with nvtx_range("moe/router"):
        gates, top_e, counts, probs_mean = native.router_topk_mean(flat, backend.router.weight, cfg.top_k, backend.aux_to_tokens)
    if not hasattr(backend, "fused_exchange"):
        from nanotitan_b200.parallel import ep_fused

        ok = flat.dtype in (torch.bfloat16, torch.float16) and flat.shape[1] % 8 == 0
        backend.fused_exchange = ep_fused.get_exchange(backend.spec.ep_group, cfg.num_experts, flat.device) if ok else None
    fused = backend.fused_exchange
    if fused is not None:
        with nvtx_range("moe/dispatch"):
            expert_in, local_offsets, packed_gate, packed_token, slot_of, ctx = fused.dispatch(flat, gates, top_e, counts)
        with nvtx_range("moe/expert_compute"):
            expert_out = backend.experts(expert_in, local_offsets)
        with nvtx_range("moe/return"):
            returned = fused.gather_back(expert_out, ctx)
    else:
        with nvtx_range("moe/pack_tokens"):
            packed_x, packed_gate, packed_token, _, _, slot_of = native.pack(flat, gates, top_e, counts)
        with nvtx_range("moe/dispatch"):
            expert_in, local_offsets, ctx = _nccl_exchange(backend, packed_x, counts)
        with nvtx_range("moe/expert_compute"):
            expert_out = backend.experts(expert_in, local_offsets)
        with nvtx_range("moe/return"):
            returned = _nccl_return(expert_out, ctx)
    with nvtx_range("moe/combine_tokens"):
        out = native.combine(returned, packed_gate, packed_token, slot_of, flat.shape[0], residual)
    return out, counts, probs_mean
