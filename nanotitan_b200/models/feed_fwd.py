"""Feed-forward modules: dense SwiGLU `FFN`, stacked SwiGLU experts, and the `MoE` layer.

Parameter names / shapes / initialisers follow the reference (src/model/feed_fwd.py:12-152):
experts are three stacked tensors `W_gate, W_val: [E_loc, d, f]`, `W_out: [E_loc, f, d]`,
the router is a bias-free Linear kept in `moe_router_dtype`.  `moe_backend = "cuda"`
selects the fused sm_100a path, `"torch"` the PyTorch-op path (also the only one on CPU).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from nanotitan_b200.models.utils import ModelShardSpec
from nanotitan_b200.utils import resolve_dtype


class FFN(nn.Module):
    """Dense SwiGLU block: W_out(silu(W_gate x) * W_val x)."""

    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        dtype = resolve_dtype(cfg.dtype)
        self.W_gate = nn.Linear(cfg.d_model, cfg.ffn_in, dtype=dtype, bias=False)
        self.W_val = nn.Linear(cfg.d_model, cfg.ffn_in, dtype=dtype, bias=False)
        self.W_out = nn.Linear(cfg.ffn_in, cfg.d_model, dtype=dtype, bias=False)
        self.silu = nn.SiLU()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.W_out(self.silu(self.W_gate(x)) * self.W_val(x))

    def parameter_count(self) -> int:
        return sum(p.numel() for p in self.parameters())


class ExpertFFN(nn.Module):
    """The local slice of the SwiGLU experts, applied to expert-major packed rows."""

    def __init__(self, cfg, spec: ModelShardSpec):
        super().__init__()
        self.cfg = cfg
        self.spec = spec
        dtype = resolve_dtype(cfg.dtype)
        n = spec.per_rank_expert
        self.W_gate = nn.Parameter(torch.empty(n, cfg.d_model, cfg.ffn_in, dtype=dtype))
        self.W_val = nn.Parameter(torch.empty(n, cfg.d_model, cfg.ffn_in, dtype=dtype))
        self.W_out = nn.Parameter(torch.empty(n, cfg.ffn_in, cfg.d_model, dtype=dtype))
        self.silu = nn.SiLU()
        self._reset_parameters()

    def _reset_parameters(self) -> None:
        for w in (self.W_gate, self.W_val, self.W_out):
            nn.init.kaiming_normal_(w, mode="fan_in", nonlinearity="relu")

    def forward(self, packed_X: torch.Tensor, expert_offset: torch.Tensor) -> torch.Tensor:
        from nanotitan_b200.ops import moe as moe_ops

        return moe_ops.swiglu_experts(
            packed_X, self.W_gate, self.W_val, self.W_out, expert_offset,
            native=(self.cfg.moe_backend == "cuda"),
        )

    def parameter_count(self) -> int:
        return sum(p.numel() for p in self.parameters())


class MoE(nn.Module):
    def __init__(self, cfg, spec: ModelShardSpec):
        super().__init__()
        self.cfg = cfg
        self.spec = spec
        self.experts = ExpertFFN(cfg, spec)
        self.router = nn.Linear(
            cfg.d_model, cfg.num_experts, bias=False, dtype=resolve_dtype(cfg.moe_router_dtype)
        )
        from nanotitan_b200.models.cuda_backend import CUDAMoEBackend
        from nanotitan_b200.models.torch_backend import TorchMoEBackend

        backend_cls = CUDAMoEBackend if cfg.moe_backend == "cuda" else TorchMoEBackend
        self.moe_backend = backend_cls(cfg, self.experts, self.router, spec)

    def active_parameter_count(self):
        router = sum(p.numel() for p in self.router.parameters())
        return router + self.cfg.top_k * (self.experts.parameter_count() / self.cfg.num_experts)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> tuple:
        return self.moe_backend.forward(x, residual)
