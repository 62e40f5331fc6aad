"""Functional ops of the model.

Every op has one CUDA implementation (autograd Functions over the `nanotitan_cuda`
kernels, in `nanotitan_b200.ops.native`) used for GPU tensors, and one plain-PyTorch
statement (`nanotitan_b200.ops.reference`) used on CPU and as the test oracle.
`NT_DISABLE_NATIVE=op1,op2` (or `all`) routes the named ops of GPU tensors through
the PyTorch statement instead; it exists to bisect numerics, not as a backend.
"""
from __future__ import annotations

import os

import torch

from nanotitan_b200.ops import reference as ref

_NATIVE_DTYPES = (torch.bfloat16, torch.float16)


def _disabled() -> set[str]:
    return {s.strip() for s in os.environ.get("NT_DISABLE_NATIVE", "").split(",") if s.strip()}


def use_native(op: str, *tensors: torch.Tensor, any_dtype: bool = False) -> bool:
    t = tensors[0]
    if not t.is_cuda:
        return False
    off = _disabled()
    if "all" in off or op in off:
        return False
    return any_dtype or t.dtype in _NATIVE_DTYPES


def layer_norm(x, gamma, beta, eps: float = 1e-8):
    if use_native("layer_norm", x, any_dtype=True):
        from nanotitan_b200.ops import native

        return native.layer_norm(x, gamma, beta, eps)
    return ref.layer_norm(x, gamma, beta, eps)


def layer_norm_residual(x, gamma, beta, eps: float = 1e-8):
    """(LayerNorm(x), x) for `x + f(LayerNorm(x))`: pass the second value on as the residual and
    the two gradients of x are summed inside the LayerNorm-backward kernel."""
    if use_native("layer_norm", x, any_dtype=True):
        from nanotitan_b200.ops import native

        return native.layer_norm_residual(x, gamma, beta, eps)
    return ref.layer_norm(x, gamma, beta, eps), x


def linear(x, w, residual=None):
    """y = x @ w (+ residual); w is [in, out]."""
    if use_native("linear", x):
        from nanotitan_b200.ops import native

        return native.linear(x, w, residual)
    return ref.linear(x, w, residual)


def causal_attention(q, k, v, scale=None):
    """q, k, v: [B, S, H, Dh] (any strides with a contiguous last dim)."""
    if use_native("attention", q):
        from nanotitan_b200.ops import native

        return native.causal_attention(q, k, v, scale)
    return ref.causal_attention(q, k, v, scale)


def qkv_attention(x, wq, wk, wv, heads: int, d_head: int, scale: float):
    """x [B, S, d] -> causal multi-head attention context [B, S, H*Dh] (q/k/v projections fused)."""
    if use_native("attention", x):
        from nanotitan_b200.ops import native

        return native.qkv_attention(x, wq, wk, wv, heads, d_head, scale)
    b, s, _ = x.shape
    q, k, v = (ref.linear(x, w).view(b, s, heads, d_head) for w in (wq, wk, wv))
    return ref.causal_attention(q, k, v, scale).reshape(b, s, heads * d_head)


def cross_entropy(logits, targets):
    if use_native("cross_entropy", logits, any_dtype=True):
        from nanotitan_b200.ops import native

        return native.cross_entropy(logits, targets)
    return ref.cross_entropy(logits, targets)


def linear_cross_entropy(x, w_unembed, targets):
    """Mean CE of (x @ w_unembed.T) against targets without keeping fp32 logits."""
    if use_native("linear_cross_entropy", x):
        from nanotitan_b200.ops import native

        return native.linear_cross_entropy(x, w_unembed, targets)
    return ref.linear_cross_entropy(x, w_unembed, targets)


__all__ = [
    "ref",
    "use_native",
    "layer_norm",
    "layer_norm_residual",
    "linear",
    "causal_attention",
    "qkv_attention",
    "cross_entropy",
    "linear_cross_entropy",
]
