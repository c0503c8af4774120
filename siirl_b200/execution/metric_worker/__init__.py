from .metric_worker import MetricClient, MetricWorker, merge_rank_metrics  # noqa: F401
