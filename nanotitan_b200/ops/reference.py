"""Plain-PyTorch statements of every op the CUDA kernels implement.

These are the numerics oracles of the kernel tests and the code path on CPU.  They
are written for clarity, in fp32 where the kernels accumulate in fp32, and they are
differentiable through autograd so a kernel's backward can be checked against
`torch.autograd.grad` of the oracle.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-8):
    """Biased-variance LayerNorm, eps inside the sqrt (reference: src/model/model.py:99-105)."""
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, keepdim=True, correction=0)
    y = (xf - mean) * torch.rsqrt(var + eps) * gamma.float() + beta.float()
    return y.to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None):
    """y = x @ w (+ residual) with w stored [in, out]."""
    y = x @ w
    return y if residual is None else y + residual


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None):
    """q, k, v: [B, S, H, Dh] -> [B, S, H, Dh]; softmax(QK^T * scale, causal) V in fp32."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    seq = q.shape[1]
    keep = torch.ones(seq, seq, dtype=torch.bool, device=q.device).tril()
    p = s.masked_fill(~keep, float("-inf")).softmax(dim=-1)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


def router_topk(x: torch.Tensor, router_w: torch.Tensor, top_k: int):
    """fp32 router: logits -> softmax -> top-k -> renormalise.

    Returns (gates [T,k] fp32, expert ids [T,k] int64, probs [T,E] fp32)
    (reference: src/model/torch_backend.py:33-40).
    """
    logits = x.to(router_w.dtype) @ router_w.t()
    probs = logits.softmax(dim=-1)
    top_p, top_e = torch.topk(probs, k=top_k, dim=-1)
    gates = top_p / top_p.sum(dim=-1, keepdim=True)
    return gates, top_e, probs


def expert_counts(top_e: torch.Tensor, num_experts: int) -> torch.Tensor:
    return torch.bincount(top_e.reshape(-1), minlength=num_experts)


def offsets_from_counts(counts: torch.Tensor) -> torch.Tensor:
    off = torch.zeros(counts.numel() + 1, dtype=counts.dtype, device=counts.device)
    off[1:] = torch.cumsum(counts, dim=0)
    return off


def pack_plan(top_e: torch.Tensor, num_experts: int):
    """Deterministic expert-major order: within an expert, ascending token id.

    Returns (slot_of [T,k] position of each assignment in packed order,
             packed_token [A], packed_k [A] which of the token's k choices, counts [E]).
    """
    tokens, k = top_e.shape
    flat = top_e.reshape(-1)
    order = torch.sort(flat, stable=True).indices  # assignment index a = t*k + j
    slot_of = torch.empty_like(order)
    slot_of[order] = torch.arange(order.numel(), device=order.device)
    return slot_of.view(tokens, k), order // k, order % k, expert_counts(top_e, num_experts)


def pack_tokens(x: torch.Tensor, gates: torch.Tensor, top_e: torch.Tensor, num_experts: int):
    """Gather token rows into expert-major order.

    Returns (packed_x [A,d], packed_token [A], packed_expert [A], packed_gate [A], counts [E]).
    """
    _, packed_token, packed_k, counts = pack_plan(top_e, num_experts)
    packed_x = x[packed_token]
    packed_gate = gates[packed_token, packed_k]
    packed_expert = top_e[packed_token, packed_k]
    return packed_x, packed_token, packed_expert, packed_gate, counts


def combine_tokens(y: torch.Tensor, packed_token: torch.Tensor, packed_gate: torch.Tensor,
                   num_tokens: int, out_dtype: torch.dtype | None = None):
    """out[t] = sum over assignments a of token t of gate[a] * y[a], fp32 accumulate."""
    out = torch.zeros(num_tokens, y.shape[1], dtype=torch.float32, device=y.device)
    out.index_add_(0, packed_token.long(), y.float() * packed_gate.float().unsqueeze(1))
    return out.to(out_dtype or y.dtype)


def grouped_gemm(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor):
    """out[r] = x[r] @ w[e] for rows r in [offsets[e], offsets[e+1])."""
    bounds = offsets.tolist()
    out = x.new_zeros(x.shape[0], w.shape[2])
    for e in range(w.shape[0]):
        lo, hi = bounds[e], bounds[e + 1]
        if hi > lo:
            out[lo:hi] = x[lo:hi] @ w[e]
    return out


def swiglu_experts(x, w_gate, w_val, w_out, offsets):
    """SwiGLU expert FFN over packed rows (reference: src/model/feed_fwd.py:80-112)."""
    bounds = offsets.tolist()
    out = x.new_zeros(x.shape[0], w_out.shape[2])
    for e in range(w_gate.shape[0]):
        lo, hi = bounds[e], bounds[e + 1]
        if hi > lo:
            xe = x[lo:hi]
            out[lo:hi] = (F.silu(xe @ w_gate[e]) * (xe @ w_val[e])) @ w_out[e]
    return out


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor):
    """Mean token cross-entropy in fp32."""
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), targets.reshape(-1))


def linear_cross_entropy(x: torch.Tensor, w_unembed: torch.Tensor, targets: torch.Tensor):
    """Unembed (weight stored [vocab, d], nn.Linear convention) followed by mean CE."""
    return cross_entropy(x @ w_unembed.t(), targets)


def adamw_step(p, g, m, v, step: int, lr: float, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.1):
    """One decoupled-weight-decay Adam update on fp32 tensors, in place (torch.optim.AdamW math)."""
    p.mul_(1.0 - lr * wd)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1**step
    bc2 = 1.0 - beta2**step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
    return p
