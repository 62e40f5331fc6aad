from nanotitan_b200.parallel.reducer import ReducerV1  # noqa: F401
