"""Recipe base classes (cf. fairseq2 ``recipe/base.py:68-366``).

A ``Recipe`` declares its config class and builds a ``Task`` from a
``RecipeContext``. The context lazily creates everything a recipe needs from
the validated config: gangs, device, output/checkpoint directories, the model
(bootstrapped from an asset card, a path or a family/arch, then wrapped for
data parallelism), optimizer, LR scheduler, metric recorders, profiler,
checkpoint manager and the trainer itself.
"""
from __future__ import annotations

import os
from abc import ABC, abstractmethod
from dataclasses import is_dataclass
from datetime import timedelta
from pathlib import Path
from typing import Any, Mapping

import torch
from torch.nn import Module
from torch.optim import Optimizer

from fairseq2_b200.assets import AssetNotFoundError, AssetStore, FileAssetMetadataProvider, get_asset_store
from fairseq2_b200.checkpoint import CheckpointManager, save_model_metadata
from fairseq2_b200.device import get_default_device
from fairseq2_b200.gang import Gangs, create_fsdp_gangs, create_parallel_gangs, setup_root_gang
from fairseq2_b200.logging import log
from fairseq2_b200.metrics.recorders import (CompositeMetricRecorder, JsonlMetricRecorder, LogMetricRecorder,
                                             MetricRecorder, TensorBoardRecorder, WandbRecorder)
from fairseq2_b200.models.family import (ModelFamily, UnknownModelArchitectureError, UnknownModelFamilyError,
                                         get_model_family)
from fairseq2_b200.nn.data_parallel import DataParallelFacade
from fairseq2_b200.optim import (AdamW, CosineAnnealingLR, MyleLR, NoamLR, NoopFloat16LossScaler, PassthroughLR,
                                 PolynomialDecayLR, StandardFloat16LossScaler, TriStageLR)
from fairseq2_b200.parallel.ddp import DDP
from fairseq2_b200.parallel.fsdp import FSDP
from fairseq2_b200.profilers import NoopProfiler, Profiler, TorchProfiler
from fairseq2_b200.recipe.config import (CommonSection, GangSection, LRSchedulerSection, ModelSection,
                                         OptimizerSection, ReferenceModelSection, RegimeSection, TrainerSection)
from fairseq2_b200.recipe.error import (FSDPNotSupportedError, GangTopologyError, ModelArchitectureNotKnownError,
                                        ModelFamilyNotKnownError, ModelNotKnownError)
from fairseq2_b200.recipe.optim import create_param_groups
from fairseq2_b200.task import Task
from fairseq2_b200.trainer import Trainer, TrainUnit, Validator
from fairseq2_b200.utils.device_stat import create_device_stat_tracker
from fairseq2_b200.utils.gc import CPythonGarbageCollector, NoopGarbageCollector
from fairseq2_b200.utils.structured import unstructure


class Recipe(ABC):
    """A runnable job description. Subclasses set ``config_kls`` and implement ``create_task``."""

    @property
    @abstractmethod
    def config_kls(self) -> type: ...

    @abstractmethod
    def create_task(self, context: "RecipeContext") -> Task: ...

    def register(self, context: "RecipeContext") -> None:
        """Hook to register recipe-specific families/components before the config is used."""

    def setup_model(self, context: "RecipeContext", model: Module, newly_initialized: bool) -> Module:
        """Hook to edit the bare model (freeze layers, add heads) before wrapping."""
        return model

    def setup_reference_model(self, context: "RecipeContext", model: Module) -> Module:
        return model

    @property
    def has_static_autograd_graph(self) -> bool:
        return True


class TrainRecipe(Recipe):
    pass


class EvalRecipe(Recipe):
    pass


class GenerationRecipe(Recipe):
    pass


class RecipeModel:
    """The model of a recipe: the wrapped (data-parallel) module, the bare module, family and config."""

    def __init__(self, dp_module: Module, base_module: Module, family: ModelFamily[Any, Any], config: Any,
                 newly_initialized: bool) -> None:
        self.module, self.base_module, self.family, self.config = dp_module, base_module, family, config
        self.newly_initialized = newly_initialized
        self.facade = DataParallelFacade(dp_module)


class RecipeDataset:
    """A dataset as a recipe sees it (cf. fairseq2 ``recipe/dataset.py:17-44``; kept for recipes written against
    the older context API): the opened dataset with the config and family it came from."""

    def __init__(self, inner_dataset: object, config: object, family: object) -> None:
        self._inner, self._config, self._family = inner_dataset, config, family

    def as_(self, kls: type) -> Any:
        if not isinstance(self._inner, kls):
            raise TypeError(f"Dataset is expected to be of type `{kls}`, but is of type `{type(self._inner)}` instead.")
        return self._inner

    @property
    def config(self) -> object:
        return self._config

    @property
    def family(self) -> object:
        return self._family


class RecipeTokenizer:
    """A tokenizer as a recipe sees it (cf. fairseq2 ``recipe/tokenizer.py:26-82``): delegates the ``Tokenizer``
    interface to the loaded tokenizer and carries its config and family."""

    def __init__(self, inner_tokenizer: Any, config: object, family: object) -> None:
        self._inner, self._config, self._family = inner_tokenizer, config, family

    def create_encoder(self, *, task: str | None = None, lang: str | None = None, mode: str | None = None,
                       device: Any = None, pin_memory: bool = False) -> Any:
        return self._inner.create_encoder(task=task, lang=lang, mode=mode, device=device, pin_memory=pin_memory)

    def create_raw_encoder(self, *, device: Any = None, pin_memory: bool = False) -> Any:
        return self._inner.create_raw_encoder(device=device, pin_memory=pin_memory)

    def create_decoder(self, *, skip_special_tokens: bool = False) -> Any:
        return self._inner.create_decoder(skip_special_tokens=skip_special_tokens)

    def as_(self, kls: type) -> Any:
        if not isinstance(self._inner, kls):
            raise TypeError(
                f"Tokenizer is expected to be of type `{kls}`, but is of type `{type(self._inner)}` instead.")
        return self._inner

    @property
    def config(self) -> object:
        return self._config

    @property
    def family(self) -> object:
        return self._family

    @property
    def vocab_info(self) -> Any:
        return self._inner.vocab_info


class RecipeContext:
    def __init__(self, config: Any, output_dir: Path, *, checkpoint_dir: Path | None = None,
                 gangs: Gangs | None = None) -> None:
        self.config = config
        self.output_dir = output_dir
        self.checkpoint_dir = checkpoint_dir or output_dir / "checkpoints"
        self._gangs = gangs
        self._store: AssetStore | None = None
        self._ckpt: CheckpointManager | None = None
        self._model: RecipeModel | None = None

    # ---------------------------------------------------------------- sections
    def _section(self, name: str, kls: type) -> Any:
        v = getattr(self.config, name, None)
        if v is None:
            return kls()
        return v

    @property
    def common(self) -> CommonSection:
        return self._section("common", CommonSection)

    # ------------------------------------------------------------------- gangs
    @property
    def gangs(self) -> Gangs:
        if self._gangs is None:
            gs: GangSection = self._section("gang", GangSection)
            ts: TrainerSection = self._section("trainer", TrainerSection)
            device = get_default_device()
            root = setup_root_gang(device, timeout=timedelta(minutes=gs.timeout), high_priority=gs.high_priority,
                                   collectives=gs.collectives)
            if root.size % gs.tensor_parallel_size != 0:
                raise GangTopologyError(root.size, gs.tensor_parallel_size)
            gangs = create_parallel_gangs(root, tp_size=gs.tensor_parallel_size)
            if ts.data_parallelism == "fsdp":
                if ts.fsdp.hybrid:
                    local = int(os.environ.get("LOCAL_WORLD_SIZE", "1"))
                    gangs = create_fsdp_gangs(gangs, intra_node_size=local)
                else:
                    gangs = create_fsdp_gangs(gangs)
            log.info("Gangs: world={} dp={} (rdp={} sdp={}) tp={} device={}", root.size, gangs.dp.size,
                     gangs.rdp.size, gangs.sdp.size, gangs.tp.size, device)
            root.barrier()   # warm-up: communicators are created before the first training step
            self._gangs = gangs
        return self._gangs

    @property
    def device(self) -> torch.device:
        return self.gangs.root.device

    # ------------------------------------------------------------------ assets
    @property
    def asset_store(self) -> AssetStore:
        if self._store is None:
            store = get_asset_store()
            for p in self.common.assets.extra_paths:
                store.add_provider(FileAssetMetadataProvider(Path(p)))
            prev = self.common.assets.prev_checkpoint_dir
            if prev is not None:
                from fairseq2_b200.assets import register_checkpoint_models

                register_checkpoint_models(store, Path(prev))
            self._store = store
        return self._store

    # ------------------------------------------------------------- checkpoints
    @property
    def checkpoint_manager(self) -> CheckpointManager:
        if self._ckpt is None:
            self._ckpt = CheckpointManager(self.checkpoint_dir, self.gangs)
        return self._ckpt

    # ------------------------------------------------------------------- model
    def bootstrap_model(self, section_name: str = "model", recipe: Recipe | None = None, *,
                        train: bool = True) -> RecipeModel:
        """Creates/loads the model of ``config.<section_name>`` and wraps it for data parallelism."""
        ms: ModelSection = getattr(self.config, section_name)
        ts: TrainerSection = self._section("trainer", TrainerSection)
        gangs = self.gangs
        store = self.asset_store
        has_ckpt = train and self.checkpoint_manager.has_checkpoint(exclude_model_only=True)
        card = None
        if ms.name is not None and ms.path is None:
            try:
                card = store.retrieve_card(ms.name)
            except AssetNotFoundError:
                raise ModelNotKnownError(ms.name) from None
            fam_name = card.maybe_get_field("model_family", str) or ms.family
        else:
            fam_name = ms.family
        if fam_name is None:
            raise ModelFamilyNotKnownError("The model family cannot be determined; set `model.family`.")
        try:
            family = get_model_family(fam_name)
        except UnknownModelFamilyError as ex:
            raise ModelFamilyNotKnownError(str(ex)) from None
        try:
            if card is not None:
                config = family.get_model_config(card, ms.config_overrides)
                if ms.arch is not None:
                    config = family.get_arch_config(ms.arch)
                    if ms.config_overrides:
                        config = family.apply_config_overrides(config, ms.config_overrides)
            else:
                config = family.get_arch_config(ms.arch)
                if ms.config_overrides:
                    config = family.apply_config_overrides(config, ms.config_overrides)
        except UnknownModelArchitectureError as ex:
            raise ModelArchitectureNotKnownError(str(ex)) from None

        from fairseq2_b200.parallel.tp import sequence_parallel

        gsec: GangSection = self._section("gang", GangSection)
        use_fsdp = train and ts.data_parallelism == "fsdp" and gangs.dp.size >= 1
        # With token-sharded activations every parameter that is replicated over the tensor-parallel gang (norm
        # weights, biases of row projections) only sees its rank's tokens: its gradient is a partial sum that the
        # flat-unit engine adds up over the gang. The bucketed DDP wrapper and a bare module do not, so those
        # configurations keep replicated activations.
        mp = ts.mixed_precision
        flat_units = use_fsdp or (train and self.device.type == "cuda" and mp.mode in ("static", "auto")
                                  and mp.dtype == torch.bfloat16 and family.supports_fsdp and ts.ddp_flat_units)
        want_sp = train and gangs.tp.size > 1 and gsec.sequence_parallel and family.supports_sequence_parallel
        if want_sp and not flat_units:
            log.info("Sequence-parallel activations need the flat-unit data-parallel engine (`trainer.data_parallelism: "
                     "fsdp`, or bf16 `ddp` on GPUs); this run keeps replicated activations.")
        seq_par = sequence_parallel(want_sp and flat_units)
        static_mp = ts.mixed_precision.mode == "static" and use_fsdp
        build_dtype = ms.dtype
        load_weights = (card is not None and card.has_field("checkpoint")) or ms.path is not None
        new_init = not load_weights
        with seq_par:
            if load_weights and not has_ckpt:
                if ms.path is not None:
                    model = family.create_new_model(config, gangs, build_dtype)
                    family.load_into(model, Path(ms.path), config, gangs, mmap=ms.mmap)
                else:
                    model = family.load_model(card, gangs, build_dtype, config=config, mmap=ms.mmap, store=store)
                log.info("Model '{}' loaded.", ms.name or ms.path)
            else:
                # fresh weights (or weights that the training checkpoint will overwrite): build on the meta
                # device when FSDP will materialise it unit by unit
                model = family.create_new_model(config, gangs, build_dtype, meta=use_fsdp and family.supports_meta)
        if recipe is not None:
            model = recipe.setup_model(self, model, new_init)
        if train:
            save_model_metadata(self.checkpoint_dir, gangs, family.name, config)
        if train and ts.activation_checkpointing.mode == "layerwise" and family.layerwise_ac_applier is not None:
            family.layerwise_ac_applier(model, ts.activation_checkpointing.every_nth_layer)
        dp_module = self.wrap_data_parallel(model, family, train=train)
        self._model = RecipeModel(dp_module, model, family, config, new_init)
        n = sum(p.numel() for p in dp_module.parameters())
        log.info("Model ready: family={} local parameters={:,}", family.name, n)
        return self._model

    def wrap_data_parallel(self, model: Module, family: ModelFamily[Any, Any], *, train: bool = True) -> Module:
        ts: TrainerSection = self._section("trainer", TrainerSection)
        gangs = self.gangs
        if not train:
            if any(p.is_meta for p in model.parameters()):
                raise ValueError("An evaluation model cannot be on the meta device.")
            return model.to(self.device)
        if ts.data_parallelism == "fsdp":
            if not family.supports_fsdp:
                raise FSDPNotSupportedError()
            mp = ts.mixed_precision
            param_dtype = mp.dtype if mp.mode == "static" else torch.float32
            if self.device.type == "cpu" and param_dtype != torch.float32:
                param_dtype = torch.float32   # the CPU plumbing path trains in fp32
            policy = None if ts.fsdp.granularity == "model" else (family.fsdp_wrap_policy or None)
            if policy is None and ts.fsdp.granularity != "model":
                from fairseq2_b200.parallel.fsdp import layerwise_wrap_policy as policy  # type: ignore[no-redef]
            return FSDP(model, gangs, wrap_policy=policy, param_dtype=param_dtype, fp32_reduce=ts.fsdp.fp32_reduce,
                        reshard_after_forward=ts.fsdp.reshard_after_forward, comm=ts.fsdp.comm,
                        cpu_offload=ts.fsdp.cpu_offload, wait_limit_s=ts.fsdp.wait_limit,
                        local_module_filter=getattr(model, "fsdp_local_module_filter", None))
        mp = ts.mixed_precision
        if (self.device.type == "cuda" and mp.mode in ("static", "auto") and mp.dtype == torch.bfloat16
                and family.supports_fsdp and ts.ddp_flat_units):
            # Replicated data parallelism on flat units: bf16 compute parameters, fp32 master weights and
            # optimizer state, gradients averaged over the replicas by the in-place all-reduce kernel as each
            # unit's backward finishes, one fused optimizer launch per unit. (The reference's DDP keeps fp32
            # parameters under autocast and all-reduces fp32 buckets with NCCL, ``nn/ddp.py:30-152``.)
            policy = family.fsdp_wrap_policy or None
            if policy is None:
                from fairseq2_b200.parallel.fsdp import layerwise_wrap_policy as policy  # type: ignore[no-redef]
            return FSDP(model, gangs, wrap_policy=policy, param_dtype=torch.bfloat16, comm=ts.fsdp.comm,
                        wait_limit_s=ts.fsdp.wait_limit)
        model = model.to(self.device)
        if gangs.dp.size > 1:
            return DDP(model, gangs)
        return model

    def bootstrap_reference_model(self, section_name: str = "reference_model", recipe: Recipe | None = None) -> Module:
        """A frozen, evaluation-mode model (e.g. the reference policy of DPO)."""
        rs: ReferenceModelSection = getattr(self.config, section_name)
        ms = ModelSection(name=rs.name, path=rs.path, family=rs.family, arch=rs.arch, dtype=rs.dtype, mmap=rs.mmap)
        saved = getattr(self.config, "model", None)
        object.__setattr__(self.config, "_ref_tmp", ms)
        try:
            rm = self.bootstrap_model("_ref_tmp", None, train=False)
        finally:
            object.__delattr__(self.config, "_ref_tmp")
        module = rm.module.eval().requires_grad_(False)
        if recipe is not None:
            module = recipe.setup_reference_model(self, module)
        return module

    # ------------------------------------------------------ tokenizer/dataset
    def load_tokenizer(self, section_name: str = "tokenizer") -> Any:
        from fairseq2_b200.assets import AssetCard
        from fairseq2_b200.data.tokenizers import load_tokenizer
        from fairseq2_b200.recipe.error import TokenizerNotKnownError

        ts = getattr(self.config, section_name)
        if ts.path is not None:
            if ts.family is None:
                raise TokenizerNotKnownError(str(ts.path))
            card = AssetCard(f"{section_name}@path", {"tokenizer_family": ts.family, "tokenizer": str(ts.path)})
            return load_tokenizer(card, store=self.asset_store)
        try:
            return load_tokenizer(ts.name, store=self.asset_store)
        except AssetNotFoundError:
            raise TokenizerNotKnownError(ts.name) from None

    def open_dataset(self, kls: type | None = None, section_name: str = "dataset") -> Any:
        from fairseq2_b200.datasets.family import UnknownDatasetError, UnknownDatasetFamilyError, open_dataset
        from fairseq2_b200.recipe.error import DatasetNotKnownError

        ds = getattr(self.config, section_name)
        try:
            return open_dataset(ds.name, family=ds.family, config_overrides=ds.config_overrides,
                                store=self.asset_store, expected_kls=kls)
        except (UnknownDatasetError, UnknownDatasetFamilyError) as ex:
            raise DatasetNotKnownError(str(ex)) from None

    # --------------------------------------------------------------- optimizer
    def create_optimizer(self, model: RecipeModel | Module) -> Optimizer:
        section: OptimizerSection = self._section("optimizer", OptimizerSection)
        module = model.module if isinstance(model, RecipeModel) else model
        cfg = dict(section.config)
        groups_cfg = cfg.pop("groups", None)
        if section.name == "adamw":
            kw = {"lr": cfg.get("lr", 1e-3), "betas": tuple(cfg.get("betas", (0.9, 0.999))),
                  "eps": cfg.get("eps", 1e-8), "weight_decay": cfg.get("weight_decay", 0.0)}
            params = create_param_groups(module, groups_cfg) if groups_cfg else module.parameters()
            return AdamW(params, **kw)
        if section.name == "adafactor":
            from fairseq2_b200.optim.adafactor import Adafactor

            return Adafactor(module.parameters(), **cfg)
        if section.name == "sgd":
            return torch.optim.SGD(module.parameters(), **cfg)
        raise ValueError(f"'{section.name}' is not a known optimizer (adamw, adafactor, sgd).")

    def create_lr_scheduler(self, optimizer: Optimizer) -> Any:
        section: LRSchedulerSection = self._section("lr_scheduler", LRSchedulerSection)
        regime: RegimeSection = self._section("regime", RegimeSection)
        if section.name is None or section.name in ("none", "passthrough"):
            return PassthroughLR(optimizer)
        cfg = dict(section.config)
        num_steps = regime.num_steps
        if section.name == "cosine_annealing":
            warm = cfg.pop("num_warmup_steps", 0)
            cycle = cfg.pop("cycle_len", None)
            if cycle is None:
                if num_steps is None:
                    raise ValueError("`lr_scheduler.config.cycle_len` must be set when `regime.num_steps` is not.")
                cycle = max(num_steps - warm, 1)
            final = cfg.pop("final_lr", None)
            scale = cfg.pop("final_lr_scale", None)
            if final is None:
                base = optimizer.param_groups[0]["lr"]
                final = base * (scale if scale is not None else 0.2)
            return CosineAnnealingLR(optimizer, cycle, warm, final_lr=final, **cfg)
        if section.name == "myle":
            return MyleLR(optimizer, **cfg)
        if section.name == "noam":
            return NoamLR(optimizer, **cfg)
        if section.name == "polynomial_decay":
            cfg.setdefault("num_steps", num_steps)
            return PolynomialDecayLR(optimizer, **cfg)
        if section.name == "tri_stage":
            cfg.setdefault("num_steps", num_steps)
            cfg["stage_ratio"] = tuple(cfg.get("stage_ratio", (0.1, 0.4, 0.5)))
            return TriStageLR(optimizer, **cfg)
        raise ValueError(f"'{section.name}' is not a known LR scheduler.")

    # ----------------------------------------------------------------- metrics
    def create_metric_recorder(self) -> MetricRecorder:
        if self.gangs.root.rank != 0:
            return CompositeMetricRecorder([])
        recs: list[MetricRecorder] = [LogMetricRecorder()]
        mr = self.common.metric_recorders
        if mr.jsonl:
            recs.append(JsonlMetricRecorder(self.output_dir / "metrics"))
        if mr.tensorboard:
            recs.append(TensorBoardRecorder(self.output_dir / "tb"))
        if mr.wandb.enabled and mr.wandb.project:
            run_id = mr.wandb.run_id
            if run_id == "persistent":
                f = self.output_dir / "wandb_run_id"
                if f.exists():
                    run_id = f.read_text().strip()
                else:
                    import uuid

                    run_id = uuid.uuid4().hex[:8]
                    f.write_text(run_id)
            recs.append(WandbRecorder(mr.wandb.project, self.output_dir, run_id=run_id, run_name=mr.wandb.run_name,
                                      entity=mr.wandb.entity, config=unstructure(self.config)))
        return CompositeMetricRecorder(recs)

    def create_profiler(self) -> Profiler:
        ps = self.common.profilers
        if not ps.enabled:
            return NoopProfiler()
        return TorchProfiler(ps.skip_n_steps, ps.wait_n_steps, ps.num_warmup_steps, ps.num_active_steps, ps.repeat,
                             self.output_dir / "tb", self.gangs.root.rank)

    # -------------------------------------------------------------- generation
    def create_seq_generator(self, model: RecipeModel | Module, tokenizer: Any,
                             section_name: str = "seq_generator") -> Any:
        """Builds the sampling or beam-search generator described by ``config.<section_name>``."""
        from fairseq2_b200.generation import (BeamSearchSequenceGenerator, SamplingSequenceGenerator,
                                              StandardBeamSearchAlgorithm, TopKSampler, TopPSampler)
        from fairseq2_b200.recipe.config import BeamSearchConfig, SamplingConfig, SequenceGeneratorSection
        from fairseq2_b200.utils.structured import structure

        section = getattr(self.config, section_name, None) or SequenceGeneratorSection()
        module = model.module if isinstance(model, RecipeModel) else model
        vi = tokenizer.vocab_info
        if vi.eos_idx is None:
            raise ValueError("The tokenizer must define an end-of-sequence symbol for generation.")
        if section.name == "sampling":
            sc: SamplingConfig = structure(dict(section.config), SamplingConfig)
            if sc.sampler.name == "top-p":
                sampler: Any = TopPSampler(float(sc.sampler.config.get("p", 0.9)))
            elif sc.sampler.name == "top-k":
                sampler = TopKSampler(int(sc.sampler.config.get("k", 1)))
            else:
                raise ValueError(f"'{sc.sampler.name}' is not a known sampler (top-p, top-k).")
            return SamplingSequenceGenerator(
                module, vi.eos_idx, vi.pad_idx, sampler, num_gens=sc.num_gens, min_gen_len=sc.min_gen_len,
                max_gen_len=sc.max_gen_len, max_seq_len=sc.max_seq_len, echo_prompt=sc.echo_prompt,
                compute_scores=sc.compute_scores, normalize_scores=sc.normalize_scores, temperature=sc.temperature,
                unk_penalty=sc.unk_penalty, len_penalty=sc.len_penalty, prefill_chunk_size=sc.prefill_chunk_size,
                decode_capacity_increment=sc.decode_capacity_increment, unk_idx=vi.unk_idx)
        if section.name == "beam_search":
            bc: BeamSearchConfig = structure(dict(section.config), BeamSearchConfig)
            if bc.algorithm != "standard":
                raise ValueError(f"'{bc.algorithm}' is not a known beam search algorithm (standard).")
            return BeamSearchSequenceGenerator(
                module, vi.eos_idx, vi.pad_idx, StandardBeamSearchAlgorithm(), beam_size=bc.beam_size,
                min_gen_len=bc.min_gen_len, max_gen_len=bc.max_gen_len, max_seq_len=bc.max_seq_len,
                echo_prompt=bc.echo_prompt, normalize_scores=bc.normalize_scores, temperature=bc.temperature,
                unk_penalty=bc.unk_penalty, len_penalty=bc.len_penalty, prefill_chunk_size=bc.prefill_chunk_size,
                decode_capacity_increment=bc.decode_capacity_increment, unk_idx=vi.unk_idx)
        raise ValueError(f"'{section.name}' is not a known sequence generator (sampling, beam_search).")

    def _eval_kwargs(self, section_name: str) -> dict[str, Any]:
        from fairseq2_b200.recipe.config import MixedPrecisionSection

        section = getattr(self.config, section_name, None)
        mp = section.mixed_precision if section is not None else MixedPrecisionSection(mode="off")
        return {"amp": mp.mode == "auto" and self.device.type == "cuda", "amp_dtype": mp.dtype,
                "metric_recorder": self.create_metric_recorder(),
                "device_stat_tracker": create_device_stat_tracker(self.device), "seed": self.common.seed}

    def create_evaluator(self, units: Any, data_readers: Any) -> Task:
        from fairseq2_b200.evaluator import Evaluator

        return Evaluator(list(units), list(data_readers), self.gangs, **self._eval_kwargs("evaluator"))

    def create_generator(self, unit: Any, data_reader: Any) -> Task:
        from fairseq2_b200.generator import Generator

        return Generator(unit, data_reader, self.gangs, **self._eval_kwargs("generator"))

    # ----------------------------------------------------------------- trainer
    def create_trainer(self, unit: TrainUnit[Any], data_reader: Any, validator: Validator | None = None, *,
                       optimizer: Optimizer | None = None, hg_exporter: Any | None = None) -> Trainer:
        ts: TrainerSection = self._section("trainer", TrainerSection)
        regime: RegimeSection = self._section("regime", RegimeSection)
        model = self._model
        if model is None:
            raise ValueError("`bootstrap_model()` must be called before `create_trainer()`.")
        optimizer = optimizer or self.create_optimizer(model)
        sched = self.create_lr_scheduler(optimizer)
        if hg_exporter is None and regime.export_hugging_face and model.family.hg_exporter is not None:
            from fairseq2_b200.checkpoint.hg import OutOfProcHuggingFaceExporter

            hg_exporter = OutOfProcHuggingFaceExporter(self.checkpoint_dir, self.gangs)
        gangs = self.gangs
        if ts.mixed_precision.mode != "off" and ts.mixed_precision.dtype == torch.float16:
            init, mn = ts.fp16_loss_scale
            scaler: Any = StandardFloat16LossScaler(gangs.dp, init_scale=init, min_scale=mn,
                                                    gradient_accumulation=ts.grad_accumulation.num_batches)
        else:
            scaler = None
        gc = CPythonGarbageCollector(ts.gc_every_n_steps) if ts.gc_every_n_steps else NoopGarbageCollector()
        return Trainer(
            unit=unit, data_reader=data_reader, gangs=gangs, optimizer=optimizer, lr_scheduler=sched,
            loss_scaler=scaler, max_grad_norm=ts.max_grad_norm,
            no_sync_grad_accumulation=ts.grad_accumulation.no_sync, grad_check=ts.grad_check,
            seed=self.common.seed + 3, max_num_steps=regime.num_steps, max_num_data_epochs=regime.num_data_epochs,
            validator=validator, validate_at_start=regime.validate_at_start,
            validate_after_n_steps=regime.validate_after_n_steps, validate_every_n_steps=regime.validate_every_n_steps,
            validate_every_n_data_epochs=regime.validate_every_n_data_epochs,
            checkpoint_manager=self.checkpoint_manager, checkpoint_after_n_steps=regime.checkpoint_after_n_steps,
            checkpoint_every_n_steps=regime.checkpoint_every_n_steps,
            checkpoint_every_n_data_epochs=regime.checkpoint_every_n_data_epochs,
            save_model_only=regime.save_model_only, keep_last_n_checkpoints=regime.keep_last_n_checkpoints,
            keep_best_n_checkpoints=regime.keep_best_n_checkpoints,
            keep_checkpoint_every_n_steps=regime.keep_checkpoint_every_n_steps,
            metric_recorder=self.create_metric_recorder(),
            publish_metrics_after_n_steps=regime.publish_metrics_after_n_steps,
            publish_metrics_every_n_steps=regime.publish_metrics_every_n_steps,
            publish_metrics_every_n_data_epochs=regime.publish_metrics_every_n_data_epochs,
            profiler=self.create_profiler(), garbage_collector=gc,
            device_stat_tracker=create_device_stat_tracker(self.device), anomaly_detection=ts.anomaly_detection,
            hg_exporter=hg_exporter, fuse_optimizer=ts.fuse_optimizer)
