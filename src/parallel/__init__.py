from nanotitan_b200.parallel import DataParallel, PipelineParallel, ReducerV1  # noqa: F401
