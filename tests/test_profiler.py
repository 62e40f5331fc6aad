"""The step profiler: rank 0 records the scheduled steps and leaves a trace plus a kernel summary."""
from types import SimpleNamespace

import torch

from nanotitan_b200.config import ProfilerConfig
from nanotitan_b200.profiler import NoOpProfiler, StepProfiler, build_profiler, nvtx_range


def _cfg(**over):
    base = dict(enabled=True, wait_steps=0, warmup_steps=1, active_steps=2, record_shapes=False, profile_memory=False,
                with_stack=False, with_flops=False)
    base.update(over)
    return ProfilerConfig(**base)


def test_rank_zero_records_and_writes_trace_and_summary(tmp_path):
    prof = build_profiler("run", _cfg(), SimpleNamespace(global_rank=0), log_root=str(tmp_path))
    assert isinstance(prof, StepProfiler)
    with prof as p:
        for _ in range(4):
            with nvtx_range("forward_pass"):
                torch.randn(32, 32) @ torch.randn(32, 32)
            p.step()
    out = tmp_path / "run" / "profiler"
    assert (out / "kernel_summary.txt").read_text().startswith("2 recorded step(s)")
    assert any(f.name.endswith(".pt.trace.json") for f in out.iterdir())


def test_other_ranks_and_disabled_configs_get_the_idle_object(tmp_path):
    assert isinstance(build_profiler("run", _cfg(), SimpleNamespace(global_rank=3), log_root=str(tmp_path)), NoOpProfiler)
    idle = build_profiler("run", _cfg(enabled=False), SimpleNamespace(global_rank=0), log_root=str(tmp_path))
    assert isinstance(idle, NoOpProfiler)
    with idle as p:
        p.step()
    assert not (tmp_path / "run").exists()
