"""Step metrics: typed values with a reduce op, one packed all-reduce, TensorBoard sink (plus the scalars
as `metrics.jsonl` next to the event files).

Metric names and the ScalarMetric / HistogramMetric contract follow the reference
(src/metrics.py:10-42, src/train.py:32-56).  The reference issues one float64
all-reduce plus a host read per metric; `reduce_metrics` here packs every metric
with the same reduce op into one flat float64 buffer, so a step costs at most two
collectives (SUM and MAX) whatever the layer count.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Literal

import torch
import torch.distributed as dist

ReduceOp = Literal["mean", "max", "sum", "none"]


@dataclass(frozen=True)
class ScalarMetric:
    value: float
    reduce: ReduceOp = "mean"


@dataclass(frozen=True)
class HistogramMetric:
    value: torch.Tensor
    reduce: ReduceOp = "mean"


class MetricsLogger:
    def __init__(self, run_name: str, log_root: str = "runs"):
        from torch.utils.tensorboard import SummaryWriter

        self.log_dir = Path(log_root) / run_name
        self.writer = SummaryWriter(log_dir=str(self.log_dir))
        # the scalars again as one JSON object per line, for scripts (sweeps, regression checks) that do not
        # want to parse TensorBoard event files
        self._lines = (self.log_dir / "metrics.jsonl").open("a", encoding="utf-8")

    def log(self, step: int, metrics: dict[str, float | torch.Tensor]) -> None:
        scalars = {"step": step}
        for name, value in metrics.items():
            if isinstance(value, torch.Tensor) and value.ndim > 0:
                self.writer.add_histogram(name, value, step)
            else:
                self.writer.add_scalar(name, float(value), step)
                scalars[name] = float(value)
        self._lines.write(json.dumps(scalars) + "\n")
        self._lines.flush()

    def log_config(self, config_dict: dict) -> None:
        self.writer.add_text("config", json.dumps(config_dict, indent=2, default=str), 0)

    def close(self) -> None:
        self.writer.close()
        self._lines.close()


def reduce_metrics(
    metrics: dict[str, ScalarMetric | HistogramMetric], device: torch.device, group=None
) -> dict[str, float | torch.Tensor]:
    """Reduce over `group` (default WORLD); scalars come back as float, histograms as fp32 CPU."""
    distributed = dist.is_available() and dist.is_initialized()
    world = dist.get_world_size(group) if distributed else 1
    plan: dict[str, list[tuple[str, int, tuple[int, ...]]]] = {"sum": [], "max": []}
    flats: dict[str, list[torch.Tensor]] = {"sum": [], "max": []}
    out: dict[str, float | torch.Tensor] = {}
    for name, metric in metrics.items():
        if metric.reduce not in ("sum", "mean", "max", "none"):
            raise ValueError(f"Unknown metric reduction: {metric.reduce}")
        value = torch.as_tensor(metric.value, dtype=torch.float64).detach().cpu()
        if metric.reduce == "none" or not distributed:
            out[name] = value.item() if value.ndim == 0 else value.to(torch.float32)
            continue
        key = "max" if metric.reduce == "max" else "sum"
        plan[key].append((name, value.numel(), tuple(value.shape)))
        flats[key].append(value.reshape(-1))
    for key, op in (("sum", dist.ReduceOp.SUM), ("max", dist.ReduceOp.MAX)):
        if not plan[key]:
            continue
        flat = torch.cat(flats[key]).to(device)
        dist.all_reduce(flat, op=op, group=group)
        flat = flat.cpu()
        cursor = 0
        for name, numel, shape in plan[key]:
            piece = flat[cursor : cursor + numel].reshape(shape)
            cursor += numel
            if metrics[name].reduce == "mean":
                piece = piece / world
            out[name] = piece.item() if piece.ndim == 0 else piece.to(torch.float32)
    return {name: out[name] for name in metrics}
