"""Recipe configuration sections (cf. fairseq2 ``recipe/config.py:96-1378``).

Plain dataclasses that are unstructured to dicts, merged with the YAML file and
``--config k=v`` overrides, then structured back with type checking."""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Literal

import torch

from fairseq2_b200.utils.validation import ValidationResult


@dataclass(kw_only=True)
class ModelSection:
    name: str | None = None
    path: Path | None = None
    family: str | None = None
    arch: str | None = None
    config_overrides: dict[str, Any] | None = None
    dtype: torch.dtype = torch.float32
    mmap: bool = False
    compile: bool = False

    def validate(self) -> ValidationResult:
        r = ValidationResult()
        if self.path is not None and self.family is None:
            r.add_error("`family` must be specified when `path` is specified.")
        if self.name is None and self.family is None:
            r.add_error("Either `name` or `family` must be specified.")
        return r


@dataclass(kw_only=True)
class ReferenceModelSection:
    """A frozen second model (e.g. the reference policy of preference optimization)."""

    name: str | None = None
    path: Path | None = None
    family: str | None = None
    arch: str | None = None
    dtype: torch.dtype = torch.bfloat16
    mmap: bool = False


@dataclass(kw_only=True)
class DatasetSection:
    name: str | None = None
    path: Path | None = None
    family: str | None = None
    config_overrides: dict[str, Any] | None = None


@dataclass(kw_only=True)
class TokenizerSection:
    name: str | None = None
    path: Path | None = None
    family: str | None = None


@dataclass(kw_only=True)
class GangSection:
    tensor_parallel_size: int = 1
    timeout: int = 15
    high_priority: bool = True
    monitored: bool = False
    #: kernels behind the root gang's CUDA collectives: "symm" = peer-memory kernels over a symmetric arena,
    #: "nccl", or "auto" (symm inside one NVSwitch domain, NCCL otherwise)
    collectives: Literal["auto", "nccl", "symm"] = "auto"
    #: training layout of tensor parallelism: the residual stream is sharded over the tokens between the blocks
    #: and the column / row projections all-gather / reduce-scatter inside their GEMM kernels (the model widens a
    #: batch by up to `tensor_parallel_size - 1` masked padding positions where the token count does not divide).
    #: Evaluation and generation models always keep their activations replicated.
    sequence_parallel: bool = True

    def validate(self) -> ValidationResult:
        r = ValidationResult()
        if self.tensor_parallel_size < 1:
            r.add_error("`tensor_parallel_size` must be greater than or equal to 1.")
        return r


@dataclass(kw_only=True)
class FSDPSection:
    version: Literal["v1", "v2", "native"] = "native"
    granularity: Literal["layer", "stack", "model"] = "layer"
    hybrid: bool = False
    reshard_after_forward: bool = True
    fp32_reduce: bool = True
    comm: Literal["auto", "symm", "nccl"] = "auto"
    cpu_offload: bool = False
    #: seconds a peer-memory collective waits for a peer before it gives up and the step raises
    wait_limit: float = 120.0


@dataclass(kw_only=True)
class MixedPrecisionSection:
    mode: Literal["off", "static", "auto"] = "static"
    dtype: torch.dtype = torch.bfloat16


@dataclass(kw_only=True)
class GradAccumulationSection:
    num_batches: int = 1
    no_sync: bool = False


@dataclass(kw_only=True)
class ActivationCheckpointingSection:
    mode: Literal["off", "layerwise"] = "off"
    every_nth_layer: int = 1


@dataclass(kw_only=True)
class TrainerSection:
    data_parallelism: Literal["ddp", "fsdp"] = "ddp"
    #: DDP on CUDA with bf16 mixed precision runs on flat parameter units (bf16 compute copies, fp32 master
    #: weights, fused all-reduce + optimizer kernels); ``False`` selects the bucketed fp32 DDP
    ddp_flat_units: bool = True
    fsdp: FSDPSection = field(default_factory=FSDPSection)
    mixed_precision: MixedPrecisionSection = field(default_factory=MixedPrecisionSection)
    grad_accumulation: GradAccumulationSection = field(default_factory=GradAccumulationSection)
    activation_checkpointing: ActivationCheckpointingSection = field(default_factory=ActivationCheckpointingSection)
    max_grad_norm: float | None = None
    #: without gradient clipping, loss scaling and gradient accumulation, FSDP runs each unit's optimizer step
    #: inside the unit's gradient reduce-scatter kernel; ``False`` keeps the separate optimizer launches
    fuse_optimizer: bool = True
    fp16_loss_scale: tuple[float, float] = (128.0, 0.0001)
    gc_every_n_steps: int | None = 1000
    grad_check: bool = False
    anomaly_detection: bool = False


@dataclass(kw_only=True)
class AdamWConfig:
    lr: float = 1e-3
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    impl: Literal["auto", "foreach", "fused", "naive"] = "auto"


@dataclass(kw_only=True)
class AdafactorConfig:
    """Hyper-parameters of :class:`fairseq2_b200.optim.Adafactor` (reference ``recipe/config.py:851-897``)."""

    lr: float = 1e-2
    beta2_decay: float = -0.8
    eps: tuple[float | None, float] = (None, 0.001)
    d: float = 1.0
    weight_decay: float = 0.0
    foreach: bool | None = None
    maximize: bool = False


@dataclass(kw_only=True)
class OptimizerSection:
    name: str = "adamw"
    config: dict[str, Any] = field(default_factory=dict)


@dataclass(kw_only=True)
class LRSchedulerSection:
    name: str | None = "cosine_annealing"
    config: dict[str, Any] = field(default_factory=dict)


@dataclass(kw_only=True)
class RegimeSection:
    num_steps: int | None = None
    num_data_epochs: int | None = None
    validate_at_start: bool = False
    validate_after_n_steps: int = 0
    validate_every_n_steps: int | None = None
    validate_every_n_data_epochs: int | None = None
    score_metric: str | None = None
    checkpoint_after_n_steps: int = 0
    checkpoint_every_n_steps: int | None = None
    checkpoint_every_n_data_epochs: int | None = None
    save_model_only: bool | Literal["all", "all_but_last"] = False
    export_hugging_face: bool = False
    keep_last_n_checkpoints: int | None = None
    keep_best_n_checkpoints: int | None = None
    keep_checkpoint_every_n_steps: int | None = None
    publish_metrics_after_n_steps: int = 0
    publish_metrics_every_n_steps: int | None = None
    publish_metrics_every_n_data_epochs: int | None = None

    def validate(self) -> ValidationResult:
        r = ValidationResult()
        if self.keep_best_n_checkpoints is not None and self.score_metric is None:
            r.add_error("`score_metric` must be specified when `keep_best_n_checkpoints` is specified.")
        for n in ("validate_every_n_steps", "checkpoint_every_n_steps", "publish_metrics_every_n_steps"):
            v = getattr(self, n)
            if v is not None and v <= 0:
                r.add_error(f"`{n}` must be greater than or equal to 1.")
        return r


@dataclass(kw_only=True)
class TorchSection:
    num_threads: int | None = None
    allow_tf32: bool = True
    fp16_reduced_precision: bool = True
    bf16_reduced_precision: bool = True
    default_sdpa: str = "b200"


@dataclass(kw_only=True)
class WandbSection:
    enabled: bool = False
    entity: str | None = None
    project: str | None = None
    run_id: str | None = "persistent"
    run_name: str | None = None


@dataclass(kw_only=True)
class MetricRecordersSection:
    jsonl: bool = True
    tensorboard: bool = False
    wandb: WandbSection = field(default_factory=WandbSection)


@dataclass(kw_only=True)
class TorchProfilerSection:
    enabled: bool = False
    skip_n_steps: int = 4
    wait_n_steps: int = 0
    num_warmup_steps: int = 1
    num_active_steps: int = 4
    repeat: int = 1


@dataclass(kw_only=True)
class AssetsSection:
    extra_paths: list[Path] = field(default_factory=list)
    prev_checkpoint_dir: Path | None = None


@dataclass(kw_only=True)
class CommonSection:
    torch: TorchSection = field(default_factory=TorchSection)
    metric_recorders: MetricRecordersSection = field(default_factory=MetricRecordersSection)
    profilers: TorchProfilerSection = field(default_factory=TorchProfilerSection)
    assets: AssetsSection = field(default_factory=AssetsSection)
    seed: int = 2
    debug: bool = False
    cluster: str = "auto"
    no_sweep_dir: bool = False
    sweep_format: str = "ws_{world_size}.{hash}"


@dataclass(kw_only=True)
class SamplerSection:
    name: str = "top-p"
    config: dict[str, Any] = field(default_factory=lambda: {"p": 0.9})


@dataclass(kw_only=True)
class SamplingConfig:
    sampler: SamplerSection = field(default_factory=SamplerSection)
    num_gens: int = 1
    min_gen_len: int = 1
    max_gen_len: int = 2048
    max_seq_len: int | None = None
    echo_prompt: bool = False
    compute_scores: bool = False
    normalize_scores: bool = True
    temperature: float = 1.0
    unk_penalty: float = 0.0
    len_penalty: float = 1.0
    prefill_chunk_size: int | None = 512
    decode_capacity_increment: int | None = 16


@dataclass(kw_only=True)
class BeamSearchConfig:
    algorithm: str = "standard"
    beam_size: int = 5
    min_gen_len: int = 1
    max_gen_len: int = 2048
    max_seq_len: int | None = None
    echo_prompt: bool = False
    normalize_scores: bool = True
    temperature: float = 1.0
    unk_penalty: float = 0.0
    len_penalty: float = 1.0
    prefill_chunk_size: int | None = 512
    decode_capacity_increment: int | None = 16


@dataclass(kw_only=True)
class SequenceGeneratorSection:
    name: str = "sampling"
    config: dict[str, Any] = field(default_factory=dict)


@dataclass(kw_only=True)
class EvaluatorSection:
    mixed_precision: MixedPrecisionSection = field(default_factory=MixedPrecisionSection)


@dataclass(kw_only=True)
class GeneratorSection:
    mixed_precision: MixedPrecisionSection = field(default_factory=MixedPrecisionSection)
