from nanotitan_b200.parallel.dp import DataParallel
from nanotitan_b200.parallel.pp import PipelineParallel
from nanotitan_b200.parallel.reducer import ReducerV1

__all__ = ["DataParallel", "PipelineParallel", "ReducerV1"]
