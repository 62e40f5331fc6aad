"""Import path of the reference's `src.utils`: the framework's helpers plus the three the reference
defines without ever calling them (src/utils.py:20-24, 37-40, 60-63)."""
from pathlib import Path

import torch

from nanotitan_b200.utils import *  # noqa: F401,F403
from nanotitan_b200.utils import (  # noqa: F401
    load_run_config, normalize_config_arg, reduce_scalars, resolve_dtype, seed_everything, setup_logging,
)


def setup_tensorboard(run_name: str, log_root: str = "runs"):
    from datetime import datetime

    from nanotitan_b200.metrics import MetricsLogger

    return MetricsLogger(f"{run_name}-{datetime.now():%Y%m%d-%H%M%S}", log_root=log_root)


def resolve_device(device_id: int) -> torch.device:
    return torch.device("cuda", device_id) if torch.cuda.is_available() else torch.device("cpu")


def get_profiler_trace_dir(run_name: str | None = None, log_root: str = "runs") -> Path | None:
    """`runs/<run_name>/profiler`; None without a run name (the reference's "no log directory" answer)."""
    return None if run_name is None else Path(log_root) / run_name / "profiler"
