from nanotitan_b200.parallel.dp import DataParallel  # noqa: F401
