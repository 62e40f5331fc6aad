"""Small helpers shared by the entrypoints (reference: src/utils.py)."""
from __future__ import annotations

import logging
import random
from datetime import datetime
from pathlib import Path

import torch
import torch.distributed as dist

from nanotitan_b200.config import AppConfig, load_config


def setup_logging(level: str = "INFO") -> None:
    logging.basicConfig(
        level=getattr(logging, str(level).upper(), logging.INFO),
        format="%(asctime)s | %(levelname)s | %(name)s | %(message)s",
    )


def setup_tensorboard(run_name: str, log_root: str = "runs"):
    from nanotitan_b200.metrics import MetricsLogger

    stamp = datetime.now().strftime("%Y%m%d-%H%M%S")
    return MetricsLogger(f"{run_name}-{stamp}", log_root=log_root)


def normalize_config_arg(config_arg: str) -> str:
    """Launcher style allows ``@path.toml``; strip the marker."""
    return config_arg[1:] if config_arg.startswith("@") else config_arg


def load_run_config(config_arg: str) -> AppConfig:
    return load_config(normalize_config_arg(config_arg))


def resolve_device(device_id: int) -> torch.device:
    return torch.device(f"cuda:{device_id}") if torch.cuda.is_available() else torch.device("cpu")


def seed_everything(seed: int) -> None:
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def reduce_scalars(scalar_tensor: torch.Tensor, pp_group) -> None:
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(scalar_tensor, op=dist.ReduceOp.SUM, group=pp_group)


def resolve_dtype(dtype):
    """'bfloat16' -> torch.bfloat16; torch dtypes and None pass through."""
    if dtype is None or isinstance(dtype, torch.dtype):
        return dtype
    return getattr(torch, dtype)


def get_profiler_trace_dir(run_name: str, log_root: str = "runs") -> Path:
    return Path(log_root) / run_name / "profiler"
