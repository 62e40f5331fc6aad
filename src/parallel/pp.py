from nanotitan_b200.parallel.pp import PipelineParallel  # noqa: F401
