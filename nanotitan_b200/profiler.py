"""torch.profiler wrapper driven by the [profiler] table (reference: src/profiler.py:39-66).

Only global rank 0 records.  Traces land in ``runs/<run_name>/profiler`` in
TensorBoard format.  `nvtx_range` marks the same named ranges for Nsight tools and
for torch.profiler at once.
"""
from __future__ import annotations

import contextlib
import logging
from pathlib import Path

import torch

from nanotitan_b200.config import ProfilerConfig

logger = logging.getLogger(__name__)


class NoOpProfiler:
    def __enter__(self) -> "NoOpProfiler":
        return self

    def __exit__(self, exc_type, exc_value, traceback) -> bool:
        return False

    def step(self) -> None:
        pass


def build_profiler(run_name: str, cfg: ProfilerConfig, dims, log_root: str = "runs"):
    if not cfg.enabled or getattr(dims, "global_rank", 0) != 0:
        return NoOpProfiler()
    trace_dir = Path(log_root) / run_name / "profiler"
    trace_dir.mkdir(parents=True, exist_ok=True)
    logger.info("Torch profiler enabled. Traces will be written to %s", trace_dir)
    activities = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        activities.append(torch.profiler.ProfilerActivity.CUDA)
    return torch.profiler.profile(
        activities=activities,
        schedule=torch.profiler.schedule(
            wait=cfg.wait_steps, warmup=cfg.warmup_steps, active=cfg.active_steps, repeat=1
        ),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(str(trace_dir)),
        record_shapes=cfg.record_shapes,
        profile_memory=cfg.profile_memory,
        with_stack=cfg.with_stack,
        with_flops=cfg.with_flops,
    )


@contextlib.contextmanager
def nvtx_range(name: str):
    """`record_function` range; also an NVTX range when CUDA is live."""
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.nvtx.range_push(name)
    try:
        with torch.profiler.record_function(name):
            yield
    finally:
        if cuda:
            torch.cuda.nvtx.range_pop()
