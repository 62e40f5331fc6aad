"""MoE building blocks: routing, pack / combine, grouped expert GEMMs, EP all-to-all.

Each function takes `native=`: True runs the sm_100a kernels (GPU tensors only),
False the PyTorch statement in `ops.reference`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from nanotitan_b200.ops import reference as ref
from nanotitan_b200.ops import use_native


def _native(flag: bool, op: str, t: torch.Tensor, any_dtype: bool = True) -> bool:
    if not flag:
        return False
    if not t.is_cuda:
        raise RuntimeError(f"{op}: moe_backend='cuda' needs GPU tensors (got {t.device})")
    return use_native(op, t, any_dtype=any_dtype)


def router_topk(x, router_w, top_k: int, native: bool = False):
    """-> (gates [T,k] fp32, expert ids [T,k], probs [T,E] fp32, counts [E])."""
    if _native(native, "router", x):
        from nanotitan_b200.ops import native as nat

        return nat.router_topk(x, router_w, top_k)
    gates, top_e, probs = ref.router_topk(x, router_w, top_k)
    return gates, top_e, probs, ref.expert_counts(top_e, router_w.shape[0])


def pack_tokens(x, gates, top_e, num_experts: int, native: bool = False):
    """-> (packed_x [A,d], packed_token [A], packed_expert [A], packed_gate [A], counts [E])."""
    if _native(native, "pack", x):
        from nanotitan_b200.ops import native as nat

        return nat.pack_tokens(x, gates, top_e, num_experts)
    return ref.pack_tokens(x, gates, top_e, num_experts)


def combine_tokens(y, packed_token, packed_gate, num_tokens: int, residual=None,
                   native: bool = False, slot_of=None):
    """out[t] = residual[t] + sum_a gate[a] * y[a]; output in y's dtype."""
    if _native(native, "combine", y):
        from nanotitan_b200.ops import native as nat

        return nat.combine_tokens(y, packed_token, packed_gate, num_tokens, residual, slot_of)
    out = ref.combine_tokens(y, packed_token, packed_gate, num_tokens)
    return out if residual is None else out + residual


def grouped_gemm(x, w, offsets, native: bool = False):
    if _native(native, "grouped_gemm", x, any_dtype=False):
        from nanotitan_b200.ops import native as nat

        return nat.grouped_gemm(x, w, offsets)
    return ref.grouped_gemm(x, w, offsets)


def swiglu_experts(x, w_gate, w_val, w_out, offsets, native: bool = False):
    if _native(native, "swiglu_experts", x, any_dtype=False):
        from nanotitan_b200.ops import native as nat

        return nat.swiglu_experts(x, w_gate, w_val, w_out, offsets)
    return ref.swiglu_experts(x, w_gate, w_val, w_out, offsets)


class AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all over rows; backward is the transposed exchange
    (reference: src/model/moe_ops.py:128-160)."""

    @staticmethod
    def forward(ctx, x, input_splits, output_splits, group):
        ctx.input_splits, ctx.output_splits, ctx.group = input_splits, output_splits, group
        out = x.new_empty((sum(output_splits), *x.shape[1:]))
        dist.all_to_all_single(
            out, x.contiguous(), output_split_sizes=output_splits,
            input_split_sizes=input_splits, group=group,
        )
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_in = grad_out.new_empty((sum(ctx.input_splits), *grad_out.shape[1:]))
        dist.all_to_all_single(
            grad_in, grad_out.contiguous(), output_split_sizes=ctx.input_splits,
            input_split_sizes=ctx.output_splits, group=ctx.group,
        )
        return grad_in, None, None, None


def all_to_all_rows(x, input_splits, output_splits, group):
    return AllToAllRows.apply(x, list(input_splits), list(output_splits), group)


def exchange_counts(send_counts: torch.Tensor, ep_size: int, group) -> torch.Tensor:
    """send_counts [E] (this rank's assignments per global expert) -> recv [ep, E_loc]:
    row s = what rank s sends to each of this rank's local experts."""
    send = send_counts.view(ep_size, -1).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def source_major_to_expert_major(recv_matrix: torch.Tensor) -> torch.Tensor:
    """Rows arrive grouped by source rank then local expert; return the gather index that
    regroups them by local expert then source rank (a stable permutation)."""
    ep, e_loc = recv_matrix.shape
    flat = recv_matrix.reshape(-1)
    cell = torch.repeat_interleave(
        torch.arange(ep * e_loc, device=flat.device), flat.long(), output_size=None
    )
    key = (cell % e_loc) * ep + cell // e_loc
    return torch.sort(key, stable=True).indices
