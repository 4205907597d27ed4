"""Metric helpers shared by recipes (cf. fairseq2 ``metrics/common.py:21-201``)."""
from __future__ import annotations

from typing import Any

from torch import Tensor

from fairseq2_b200.metrics.aggregation import Mean, Sum
from fairseq2_b200.metrics.bag import MetricBag


def update_nll_loss_metric(bag: MetricBag, loss: Tensor, num_targets: int | Tensor) -> None:
    """``nll_loss`` in bits per target (sum-reduced natural-log loss / targets / ln 2)."""
    import math

    bag.get("nll_loss", Mean).update(loss.detach() / num_targets / math.log(2), weight=num_targets)


def update_seq_batch_metrics(bag: MetricBag, num_examples: int, num_elements: int, num_target_elements: int,
                             padding: int = 0) -> None:
    bag.get("num_examples", Sum).update(num_examples)
    bag.get("num_elements", Sum).update(num_elements)
    bag.get("num_target_elements", Sum).update(num_target_elements)
    bag.get("total_num_examples", Sum).update(num_examples)
    bag.get("total_num_elements", Sum).update(num_elements)
    bag.get("total_num_target_elements", Sum).update(num_target_elements)
    bag.get("padding", Sum).update(padding)


def extend_batch_metric_values(values: dict[str, Any], num_batches: int, elapsed_time: float) -> None:
    """Derives ``batch_size``, ``elements_per_batch``, ``elements_per_second`` and ``padding_ratio``."""
    ne, nel = values.get("num_examples"), values.get("num_elements")
    if ne is not None and num_batches > 0:
        values["batch_size"] = ne / num_batches
    if nel is not None:
        if num_batches > 0:
            values["elements_per_batch"] = nel / num_batches
        if elapsed_time > 0:
            values["elements_per_second"] = nel / elapsed_time
        pad = values.get("padding")
        if pad is not None and nel + pad > 0:
            values["padding_ratio"] = pad / (nel + pad)
