from nanotitan_b200.metrics import HistogramMetric, MetricsLogger, ReduceOp, ScalarMetric, reduce_metrics  # noqa: F401
