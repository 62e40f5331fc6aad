"""Causal self-attention on GPU tensors: dispatch to the flash kernels."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def causal_attention(q, k, v, scale=None):
    """q, k, v: [B, S, H, Dh] -> [B, S, H, Dh]."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    from nanotitan_b200.ops import flash

    if flash.supported(q, k, v):
        return flash.flash_attention(q, k, v, scale)
    out = F.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, scale=scale
    )
    return out.transpose(1, 2)
