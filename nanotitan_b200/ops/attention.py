"""Causal self-attention on GPU tensors: dispatch to the tcgen05 kernels.

Shapes the kernels do not cover (head sizes other than 32 / 64, fp32 tensors) go to PyTorch's
scaled-dot-product attention, announced through `native.library_fallback` (a warning once, an error
under NT_STRICT=1); the benchmark configurations never take that branch.
"""
from __future__ import annotations

import math

import torch.nn.functional as F


def causal_attention(q, k, v, scale=None):
    """q, k, v: [B, S, H, Dh] -> [B, S, H, Dh]."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    from nanotitan_b200.ops import flash, native

    if flash.supported(q, k, v):
        return flash.flash_attention(q, k, v, scale)
    native.library_fallback("causal_attention", f"dtype {q.dtype}, head dim {q.shape[-1]}: the kernels take bf16/fp16 with head dim 32 or 64")
    out = F.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, scale=scale
    )
    return out.transpose(1, 2)
