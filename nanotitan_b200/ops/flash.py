"""tcgen05 flash-attention kernels (forward and backward) behind an autograd Function.

The reference computes attention as softmax(QK^T / sqrt(Dh) + mask) V with a stored [1, 1, S, S] boolean mask
(src/model/model.py:122-182); these kernels never form the S x S matrix.
"""
from __future__ import annotations

import torch

from nanotitan_b200.ops.ext import get_ext


def supported(q, k, v) -> bool:
    ext = get_ext()
    if not hasattr(ext, "flash_fwd"):
        return False
    return (
        q.dtype in (torch.bfloat16, torch.float16)
        and q.shape[-1] in (32, 64)
        and q.shape == k.shape == v.shape
    )


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        ext = get_ext()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse = ext.flash_fwd(q, k, v, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = get_ext().flash_bwd(dout.contiguous(), q, k, v, out, lse, ctx.scale)
        return dq, dk, dv, None


def flash_attention(q, k, v, scale):
    return _Flash.apply(q, k, v, scale)


class _FlashQKV(torch.autograd.Function):
    """Attention over a fused projection buffer qkv [B, S, 3*H*Dh] (q | k | v side by side); the
    backward kernels write dq, dk, dv straight into the thirds of one dQKV buffer."""

    @staticmethod
    def forward(ctx, qkv, heads, d_head, scale):
        b, s, _ = qkv.shape
        inner = heads * d_head
        q, k, v = (qkv[..., i * inner : (i + 1) * inner].view(b, s, heads, d_head) for i in range(3))
        out, lse = get_ext().flash_fwd(q, k, v, scale)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (heads, d_head, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        heads, d_head, scale = ctx.meta
        b, s, _ = qkv.shape
        inner = heads * d_head
        dqkv = torch.empty_like(qkv)
        q, k, v = (qkv[..., i * inner : (i + 1) * inner].view(b, s, heads, d_head) for i in range(3))
        grads = [dqkv[..., i * inner : (i + 1) * inner].view(b, s, heads, d_head) for i in range(3)]
        get_ext().flash_bwd(dout.contiguous(), q, k, v, out, lse, scale, grads)
        return dqkv, None, None, None


def flash_attention_qkv(qkv, heads, d_head, scale):
    return _FlashQKV.apply(qkv, heads, d_head, scale)
