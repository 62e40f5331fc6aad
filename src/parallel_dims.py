from nanotitan_b200.parallel_dims import ParallelDims, RankLayout, get_parallel_dims  # noqa: F401
