from nanotitan_b200.profiler import NoOpProfiler, build_profiler, nvtx_range  # noqa: F401
