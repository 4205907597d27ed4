from fairseq2_b200.metrics.aggregation import Max, Mean, Metric, Min, Sum
from fairseq2_b200.metrics.bag import MetricBag, sync_and_compute_metrics
