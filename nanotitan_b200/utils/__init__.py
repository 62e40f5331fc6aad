"""Helpers shared by the entrypoints: logging, seeding, dtype names, config arguments.

The names are the reference's (src/utils.py:13-57): `setup_logging`, `normalize_config_arg`,
`load_run_config`, `seed_everything`, `reduce_scalars`, `resolve_dtype`.  Helpers the reference
defines but never calls live only in the `src.utils` compatibility module.
"""
from __future__ import annotations

import logging
import os
import random

import torch
import torch.distributed as dist

from nanotitan_b200.config import AppConfig, load_config

__all__ = ["setup_logging", "normalize_config_arg", "load_run_config", "seed_everything", "reduce_scalars",
           "resolve_dtype", "DTYPE_NAMES"]

# accepted spellings of the three training dtypes (the TOML files use the torch names)
DTYPE_NAMES = {
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "float64": torch.float64, "fp64": torch.float64, "double": torch.float64,
}


def resolve_dtype(dtype):
    """Config spelling -> `torch.dtype`.  Dtypes and None pass through; an unknown name is an error
    here, at start-up, not at the first tensor creation."""
    if dtype is None or isinstance(dtype, torch.dtype):
        return dtype
    try:
        return DTYPE_NAMES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}; known: {sorted(DTYPE_NAMES)}") from None


def setup_logging(level: str = "INFO") -> None:
    """Root logger at `level` (a name such as "debug" or a number), each line tagged with the rank
    the launcher gave this process."""
    numeric = logging.getLevelName(str(level).upper())
    if not isinstance(numeric, int):
        numeric = int(level) if str(level).isdigit() else logging.INFO
    rank = os.environ.get("RANK")
    tag = f"rank {rank} | " if rank is not None else ""
    logging.basicConfig(level=numeric, format=f"%(asctime)s | {tag}%(levelname)s | %(name)s | %(message)s")


def normalize_config_arg(config_arg: str) -> str:
    """`@configs/x.toml` (launcher style) and `configs/x.toml` name the same file."""
    return config_arg.removeprefix("@")


def load_run_config(config_arg: str) -> AppConfig:
    return load_config(normalize_config_arg(config_arg))


def seed_everything(seed: int) -> None:
    """Same seed on every rank: replicas build identical initial weights before the first
    broadcast, as in the reference (src/train.py:94)."""
    random.seed(seed)
    torch.manual_seed(seed)  # seeds the CPU generator and every CUDA device's
    try:
        import numpy as np

        np.random.seed(seed % (1 << 32))
    except ImportError:
        pass


def reduce_scalars(scalar_tensor: torch.Tensor, pp_group) -> None:
    """In-place SUM over `pp_group` (parameter counts over the pipeline stages); a no-op without a
    process group."""
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(scalar_tensor, op=dist.ReduceOp.SUM, group=pp_group)
