"""Metric recorders: log table, JSONL files, TensorBoard, Weights & Biases and a
composite (cf. fairseq2 ``metrics/recorders/*``). Descriptors give each metric a
display name, sort priority and formatter."""
from __future__ import annotations

import json
import math
from abc import ABC, abstractmethod
from dataclasses import dataclass
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

from fairseq2_b200.logging import log


def format_as_int(v: Any) -> str:
    return f"{int(v):,}"


def format_as_float(v: Any) -> str:
    return f"{float(v):g}"


def format_as_seconds(v: Any) -> str:
    return f"{float(v):.1f}s"


def format_as_percentage(v: Any) -> str:
    return f"{float(v) * 100:.2f}%"


def format_as_byte_size(v: Any) -> str:
    x = float(v)
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if x < 1024 or unit == "TiB":
            return f"{x:.2f} {unit}"
        x /= 1024
    return f"{x:.2f}"


@dataclass(frozen=True)
class MetricDescriptor:
    name: str
    display_name: str
    priority: int
    formatter: Callable[[Any], str]
    log: bool = True
    higher_better: bool = False


_DESCRIPTORS: dict[str, MetricDescriptor] = {}


def register_metric_descriptor(d: MetricDescriptor) -> None:
    _DESCRIPTORS[d.name] = d


def get_metric_descriptor(name: str) -> MetricDescriptor | None:
    return _DESCRIPTORS.get(name)


for _d in [
    MetricDescriptor("loss", "Loss", 90, format_as_float),
    MetricDescriptor("nll_loss", "NLL Loss", 100, format_as_float),
    MetricDescriptor("ctc_loss", "CTC Loss", 100, format_as_float),
    MetricDescriptor("contrastive_loss", "Contrastive Loss", 100, format_as_float),
    MetricDescriptor("diversity_loss", "Diversity Loss", 100, format_as_float),
    MetricDescriptor("accuracy", "Accuracy", 200, format_as_percentage, higher_better=True),
    MetricDescriptor("bleu", "BLEU", 200, format_as_float, higher_better=True),
    MetricDescriptor("chrf", "chrF++", 200, format_as_float, higher_better=True),
    MetricDescriptor("wer", "WER", 200, format_as_float),
    MetricDescriptor("uer", "UER", 200, format_as_float),
    MetricDescriptor("grad_norm", "Gradient Norm", 300, format_as_float),
    MetricDescriptor("lr", "Learning Rate", 310, format_as_float),
    MetricDescriptor("data_epoch", "Data Epoch", 490, format_as_int),
    MetricDescriptor("data_time", "Data Time", 500, format_as_seconds),
    MetricDescriptor("compute_time", "Compute Time", 501, format_as_seconds),
    MetricDescriptor("lapse_time", "Lapse Time", 502, format_as_seconds),
    MetricDescriptor("total_time", "Total Time", 505, format_as_seconds),
    MetricDescriptor("wall_time", "Wall Time", 510, format_as_seconds),
    MetricDescriptor("batch_size", "Batch Size", 700, format_as_int),
    MetricDescriptor("elements_per_batch", "Elements per Batch", 701, format_as_int),
    MetricDescriptor("elements_per_second", "Elements per Second", 702, format_as_int, higher_better=True),
    MetricDescriptor("generator_elements_per_second", "Generated Elements per Second", 703, format_as_int,
                     higher_better=True),
    MetricDescriptor("num_examples", "Number of Examples", 710, format_as_int),
    MetricDescriptor("num_elements", "Number of Elements", 711, format_as_int),
    MetricDescriptor("num_target_elements", "Number of Target Elements", 712, format_as_int),
    MetricDescriptor("padding", "Padding", 713, format_as_int),
    MetricDescriptor("padding_ratio", "Padding Ratio (%)", 714, format_as_percentage),
    MetricDescriptor("total_num_examples", "Total Number of Examples", 720, format_as_int),
    MetricDescriptor("total_num_elements", "Total Number of Elements", 721, format_as_int),
    MetricDescriptor("total_num_target_elements", "Total Number of Target Elements", 722, format_as_int),
    MetricDescriptor("peak_active_mem_bytes", "Peak Active Device Memory", 920, format_as_byte_size),
    MetricDescriptor("peak_active_mem_ratio", "Peak Active Device Memory (%)", 921, format_as_percentage),
    MetricDescriptor("peak_reserved_mem_bytes", "Peak Reserved Device Memory", 925, format_as_byte_size),
    MetricDescriptor("num_alloc_retries", "Device Allocation Retries", 930, format_as_int),
]:
    register_metric_descriptor(_d)


def format_metric_value(name: str, value: Any) -> str:
    d = get_metric_descriptor(name)
    if d is None:
        return f"{value:g}" if isinstance(value, float) else str(value)
    return d.formatter(value)


class MetricRecorder(ABC):
    @abstractmethod
    def record_metric_values(self, category: str, values: Mapping[str, Any], step_nr: int | None = None) -> None: ...

    def close(self) -> None:
        pass


class NoopMetricRecorder(MetricRecorder):
    def record_metric_values(self, category: str, values: Mapping[str, Any], step_nr: int | None = None) -> None:
        pass


class CompositeMetricRecorder(MetricRecorder):
    def __init__(self, recorders: Sequence[MetricRecorder]) -> None:
        self._recorders = list(recorders)

    def record_metric_values(self, category: str, values: Mapping[str, Any], step_nr: int | None = None) -> None:
        for r in self._recorders:
            r.record_metric_values(category, values, step_nr)

    def close(self) -> None:
        for r in self._recorders:
            r.close()


def _sorted_items(values: Mapping[str, Any]) -> list[tuple[str, Any]]:
    def key(item: tuple[str, Any]) -> tuple[int, str]:
        d = get_metric_descriptor(item[0])
        return (d.priority if d else 10_000, item[0])

    return sorted(values.items(), key=key)


class LogMetricRecorder(MetricRecorder):
    def record_metric_values(self, category: str, values: Mapping[str, Any], step_nr: int | None = None) -> None:
        parts = []
        for n, v in _sorted_items(values):
            d = get_metric_descriptor(n)
            if d is not None and not d.log:
                continue
            parts.append(f"{d.display_name if d else n}: {format_metric_value(n, v)}")
        title = category.capitalize() + " Metrics"
        if step_nr is not None:
            title += f" (step {step_nr})"
        log.info("{} - {}", title, " | ".join(parts))


class JsonlMetricRecorder(MetricRecorder):
    """Appends one JSON object per publish to ``<dir>/<category>.jsonl`` with ``Time`` and ``Step``."""

    def __init__(self, output_dir: Path) -> None:
        self._dir = output_dir
        self._streams: dict[str, Any] = {}

    def record_metric_values(self, category: str, values: Mapping[str, Any], step_nr: int | None = None) -> None:
        fp = self._streams.get(category)
        if fp is None:
            path = self._dir / (category.replace("/", "_") + ".jsonl")
            path.parent.mkdir(parents=True, exist_ok=True)
            fp = path.open("a", encoding="utf-8")
            self._streams[category] = fp
        out: dict[str, Any] = {"Time": datetime.now(timezone.utc).isoformat()}
        if step_nr is not None:
            out["Step"] = step_nr
        for n, v in _sorted_items(values):
            d = get_metric_descriptor(n)
            key = d.display_name if d else n
            if hasattr(v, "tolist") and not isinstance(v, (str, bytes)):
                v = v.tolist()                      # tensors and numpy values (0-dim -> Python scalar)
            if isinstance(v, float) and not math.isfinite(v):
                v = str(v)
            out[key] = v
        fp.write(json.dumps(out) + "\n")
        fp.flush()

    def close(self) -> None:
        for fp in self._streams.values():
            fp.close()
        self._streams.clear()


class TensorBoardRecorder(MetricRecorder):
    def __init__(self, output_dir: Path) -> None:
        self._dir = output_dir
        self._writers: dict[str, Any] = {}

    def _writer(self, category: str) -> Any:
        w = self._writers.get(category)
        if w is None:
            try:
                from torch.utils.tensorboard import SummaryWriter
            except ImportError:
                log.warning("tensorboard is not installed; TensorBoard recording is disabled.")
                return None
            w = SummaryWriter(str(self._dir / category))
            self._writers[category] = w
        return w

    def record_metric_values(self, category: str, values: Mapping[str, Any], step_nr: int | None = None) -> None:
        w = self._writer(category)
        if w is None:
            return
        for n, v in values.items():
            d = get_metric_descriptor(n)
            if isinstance(v, (int, float)):
                w.add_scalar(d.display_name if d else n, v, step_nr)
        w.flush()

    def close(self) -> None:
        for w in self._writers.values():
            w.close()
        self._writers.clear()


class WandbRecorder(MetricRecorder):
    """Logs to Weights & Biases; ``run_id='persistent'`` semantics (reusing the
    id stored next to the output directory) are handled by the recipe layer."""

    def __init__(self, project: str, output_dir: Path, *, run_id: str | None = None, run_name: str | None = None,
                 entity: str | None = None, config: Mapping[str, Any] | None = None) -> None:
        try:
            import wandb
        except ImportError:
            log.warning("wandb is not installed; W&B recording is disabled.")
            self._run = None
            return
        try:
            self._run = wandb.init(project=project, entity=entity, id=run_id, name=run_name, dir=str(output_dir),
                                   config=dict(config or {}), resume="allow")
        except Exception as ex:  # noqa: BLE001 - offline boxes
            log.warning("W&B cannot be initialised ({}); recording is disabled.", ex)
            self._run = None

    def record_metric_values(self, category: str, values: Mapping[str, Any], step_nr: int | None = None) -> None:
        if self._run is None:
            return
        out = {}
        for n, v in values.items():
            d = get_metric_descriptor(n)
            out[f"{category}/{d.display_name if d else n}"] = v
        self._run.log(out, step=step_nr)

    def close(self) -> None:
        if self._run is not None:
            self._run.finish()
