"""Step profiler driven by the `[profiler]` table, and the named ranges of the hot path.

`build_profiler(run_name, cfg, dims)` has the reference's contract (src/profiler.py:39-66): a
context manager with a `.step()` method that records on global rank 0 only, after `wait_steps`
idle and `warmup_steps` warm-up steps, for `active_steps` steps, into
`runs/<run_name>/profiler` (TensorBoard traces).  On top of the trace this one also leaves
`kernel_summary.txt` in that folder: device time per kernel over the recorded steps, which is
usually the first thing looked for.  `nvtx_range` marks a named range for torch.profiler and,
when CUDA is live, for the Nsight tools.
"""
from __future__ import annotations

import contextlib
import logging
from pathlib import Path

import torch
from torch.profiler import ProfilerActivity, profile, record_function, schedule, tensorboard_trace_handler

from nanotitan_b200.config import ProfilerConfig

logger = logging.getLogger(__name__)


class _Idle:
    """What every rank but the recording one gets: same surface, no work."""

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> bool:
        return False

    def step(self) -> None:
        return None


NoOpProfiler = _Idle  # the reference's name for it


class StepProfiler:
    def __init__(self, cfg: ProfilerConfig, out_dir: Path):
        self.out_dir = out_dir
        self.out_dir.mkdir(parents=True, exist_ok=True)
        kinds = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        self._prof = profile(
            activities=kinds,
            schedule=schedule(wait=cfg.wait_steps, warmup=cfg.warmup_steps, active=cfg.active_steps, repeat=1),
            on_trace_ready=self._on_trace,
            record_shapes=cfg.record_shapes, profile_memory=cfg.profile_memory,
            with_stack=cfg.with_stack, with_flops=cfg.with_flops,
        )
        self._to_tensorboard = tensorboard_trace_handler(str(out_dir))
        self._steps = cfg.active_steps

    def _on_trace(self, prof) -> None:
        self._to_tensorboard(prof)
        try:
            table = prof.key_averages().table(sort_by="self_cuda_time_total" if torch.cuda.is_available() else "self_cpu_time_total",
                                              row_limit=60)
            (self.out_dir / "kernel_summary.txt").write_text(f"{self._steps} recorded step(s)\n{table}\n")
        except Exception as exc:  # a summary must never take the run down
            logger.warning("could not write the kernel summary: %s", exc)

    def __enter__(self):
        self._prof.__enter__()
        return self

    def __exit__(self, *exc) -> bool:
        self._prof.__exit__(*exc)
        return False

    def step(self) -> None:
        self._prof.step()


def build_profiler(run_name: str, cfg: ProfilerConfig, dims, log_root: str = "runs"):
    recording = cfg.enabled and getattr(dims, "global_rank", 0) == 0
    if not recording:
        return _Idle()
    out_dir = Path(log_root) / run_name / "profiler"
    logger.info("profiling steps %d..%d of rank 0 into %s", cfg.wait_steps + cfg.warmup_steps,
                cfg.wait_steps + cfg.warmup_steps + cfg.active_steps - 1, out_dir)
    return StepProfiler(cfg, out_dir)


@contextlib.contextmanager
def nvtx_range(name: str):
    """`record_function` range; also an NVTX range when CUDA is live."""
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.nvtx.range_push(name)
    try:
        with record_function(name):
            yield
    finally:
        if cuda:
            torch.cuda.nvtx.range_pop()
