"""Optimizer factory.

`type = "adam"` means AdamW with weight decay 0.1 on every parameter, default betas
and eps, as in the reference (src/optim.py:6-10).  On CUDA the update runs in the
framework's fused AdamW kernel over flat fp32 master/moment buffers; on CPU it is
`torch.optim.AdamW`.
"""
from __future__ import annotations

import torch

from nanotitan_b200.config import OptimizerConfig

WEIGHT_DECAY = 0.1


def setup_optimizer(cfg: OptimizerConfig, model, fused: bool | None = None):
    if cfg.type != "adam":
        raise ValueError(f"Optimizer type {cfg.type} is not supported")
    params = [p for p in model.parameters() if p.requires_grad]
    on_cuda = bool(params) and params[0].is_cuda
    if fused is None:
        fused = on_cuda
    if fused:
        from nanotitan_b200.ops.adamw import FusedAdamW

        return FusedAdamW(params, lr=cfg.lr, weight_decay=WEIGHT_DECAY)
    return torch.optim.AdamW(params, lr=cfg.lr, weight_decay=WEIGHT_DECAY)
