def sync_and_compute_collection(metrics, process_group=None, recipient_rank=0):
    return {k: m.compute() for k, m in metrics.items()}


def sync_and_compute(metric, process_group=None, recipient_rank=0):
    return metric.compute()
