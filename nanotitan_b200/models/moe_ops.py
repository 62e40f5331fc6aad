"""Autograd entry points of the MoE dispatch kernels under the reference's names
(src/model/moe_ops.py:10-37): same argument order, same return conventions."""
from __future__ import annotations

import torch

from nanotitan_b200.ops import moe as _moe


def pack_tokens_fn(X, topk_weights, topk_experts, expert_offset_cpy):
    """-> (packed_X, packed_tokenId int32, packed_expert int32, packed_topk_weights fp32).

    `expert_offset_cpy` ([E] or [E+1] exclusive offsets) only fixes the expert count:
    slots come from a deterministic scan, not from atomics on this buffer."""
    num_experts = expert_offset_cpy.numel() - 1 if expert_offset_cpy.numel() > 1 else 1
    num_experts = max(num_experts, int(topk_experts.max().item()) + 1) if topk_experts.numel() else num_experts
    px, ptok, pexp, pgate, _ = _moe.pack_tokens(
        X, topk_weights, topk_experts, num_experts, native=X.is_cuda
    )
    return px, ptok.to(torch.int32), pexp.to(torch.int32), pgate


def combine_tokens_fn(packed_expert_outputs, packed_tokenId, packed_topk_weights, num_tokens, hidden_dim):
    assert packed_expert_outputs.shape[1] == hidden_dim
    return _moe.combine_tokens(
        packed_expert_outputs, packed_tokenId, packed_topk_weights, num_tokens,
        native=packed_expert_outputs.is_cuda,
    )


def grouped_gemm_fn(X, weight, expert_offset):
    return _moe.grouped_gemm(X, weight, expert_offset, native=X.is_cuda)


def torch_backend_all_to_all(x, input_splits, output_splits, group):
    return _moe.all_to_all_rows(x, input_splits, output_splits, group)


class _ApplyOnly:
    """The reference spells these operations as `torch.autograd.Function` subclasses and callers may reach
    them as `Name.apply(...)` (src/model/moe_ops.py:40-160).  Here the autograd nodes live with the kernels
    (ops/native.py, ops/moe.py); these names keep that spelling working."""

    def __init__(self):
        raise TypeError(f"{type(self).__name__} is used through {type(self).__name__}.apply(...)")


class PackTokensFN(_ApplyOnly):
    @staticmethod
    def apply(X, topk_weights, topk_experts, expert_offset_cpy):
        return pack_tokens_fn(X, topk_weights, topk_experts, expert_offset_cpy)


class CombineTokensFN(_ApplyOnly):
    @staticmethod
    def apply(packed_expert_outputs, packed_tokenId, packed_topk_weights, num_tokens, hidden_dim):
        return combine_tokens_fn(packed_expert_outputs, packed_tokenId, packed_topk_weights, num_tokens, hidden_dim)


class GroupedGEMM_FN(_ApplyOnly):
    @staticmethod
    def apply(X, expert_offset, weight):  # note the order: offsets before weights, unlike grouped_gemm_fn
        return grouped_gemm_fn(X, weight, expert_offset)


class TorchBackendAll2ALL(_ApplyOnly):
    @staticmethod
    def apply(x, input_splits, output_splits, group):
        return torch_backend_all_to_all(x, input_splits, output_splits, group)
