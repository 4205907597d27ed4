"""Hugging Face ``transformers`` models behind this framework's model interfaces (cf. fairseq2
``models/hg/config.py:18-118``, ``hg/factory.py:73-546``, ``hg/adapter.py:28-329``, ``hg/api.py:24-178``).

``create_hg_model`` instantiates any ``transformers`` model from a local directory or hub name
(``AutoModel*`` classes, or a registered custom class); causal LMs are wrapped in
:class:`HgCausalLMAdapter`, which speaks the :class:`~fairseq2_b200.models.clm.CausalLM` contract
(batch layouts in, sum-reduced loss or logits out) so that trainers, recipes and generators work on it
unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
from torch import Tensor
from torch.nn import Module

from fairseq2_b200.models.clm import CausalLM
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.functional import cross_entropy
from fairseq2_b200.runtime.config_registry import ConfigRegistrar
from fairseq2_b200.typing import DataType

HG_FAMILY = "hg"


class HuggingFaceModelError(Exception):
    def __init__(self, model_name: str, message: str) -> None:
        super().__init__(message)
        self.model_name = model_name


@dataclass(kw_only=True)
class HuggingFaceModelConfig:
    hf_name: str = "gpt2"
    """Hub identifier or local directory."""
    model_type: str = "auto"
    """``auto``, ``causal_lm``, ``seq2seq_lm`` or ``custom``."""
    use_processor: bool = False
    device: str = "cpu"
    custom_model_class: str | None = None
    custom_processor_class: str | None = None
    trust_remote_code: bool = False
    dtype: DataType | None = None
    load_kwargs: dict[str, Any] | None = None
    enable_gradient_checkpointing: bool = False
    random_init: bool = False
    """Build from the configuration only (no weights are read); used for tests and from-scratch training."""


arch = ConfigRegistrar(HuggingFaceModelConfig)
arch("causal_lm")(lambda: HuggingFaceModelConfig(hf_name="gpt2", model_type="causal_lm"))
arch("seq2seq_lm")(lambda: HuggingFaceModelConfig(hf_name="google-t5/t5-small", model_type="seq2seq_lm"))
arch("auto")(lambda: HuggingFaceModelConfig(hf_name="bert-base-uncased", model_type="auto"))
arch("custom")(lambda: HuggingFaceModelConfig(hf_name="Qwen/Qwen2.5-Omni-3B", model_type="custom"))

# config class name -> {"model": ..., "tokenizer": ..., "processor": ...} for architectures the Auto classes miss
_CUSTOM_CLASSES: dict[str, dict[str, Any]] = {}


def register_hg_model_class(config_class_name: str, model_class: type | str, tokenizer_class: type | str | None = None,
                            processor_class: type | str | None = None) -> None:
    entry: dict[str, Any] = {"model": model_class}
    if tokenizer_class is not None:
        entry["tokenizer"] = tokenizer_class
    if processor_class is not None:
        entry["processor"] = processor_class
    _CUSTOM_CLASSES[config_class_name] = entry


def _transformers() -> Any:
    try:
        import transformers
    except ImportError as ex:
        raise HuggingFaceModelError("-", "The `transformers` package is required for the 'hg' model family.") from ex
    return transformers


def _resolve_class(cls: type | str) -> Any:
    if not isinstance(cls, str):
        return cls
    tf = _transformers()
    try:
        return getattr(tf, cls)
    except AttributeError:
        raise HuggingFaceModelError(cls, f"`transformers` has no class named '{cls}'.") from None


def _auto_class(config: HuggingFaceModelConfig, hf_config: Any) -> Any:
    tf = _transformers()
    if config.model_type == "causal_lm":
        return tf.AutoModelForCausalLM
    if config.model_type == "seq2seq_lm":
        return tf.AutoModelForSeq2SeqLM
    if config.model_type == "auto":
        archs = getattr(hf_config, "architectures", None) or []
        if any(a.endswith("ForCausalLM") or a.endswith("LMHeadModel") for a in archs):
            return tf.AutoModelForCausalLM
        if any(a.endswith("ForConditionalGeneration") for a in archs) and getattr(hf_config, "is_encoder_decoder", False):
            return tf.AutoModelForSeq2SeqLM
        return tf.AutoModel
    raise HuggingFaceModelError(config.hf_name, f"`model_type` must be 'auto', 'causal_lm', 'seq2seq_lm' or 'custom', "
                                                f"but is '{config.model_type}' instead.")


def create_hg_model(config: HuggingFaceModelConfig, gangs: object | None = None, *, hf_config: Any | None = None) -> Module:
    """Instantiates the model described by ``config``. ``hf_config`` overrides the configuration that would be
    read from ``config.hf_name`` (which then does not need to exist when ``random_init`` is set)."""
    tf = _transformers()
    name = config.hf_name
    kwargs: dict[str, Any] = dict(config.load_kwargs or {})
    if config.dtype is not None:
        kwargs["torch_dtype"] = config.dtype
    if config.trust_remote_code:
        kwargs["trust_remote_code"] = True
    try:
        if hf_config is None:
            hf_config = tf.AutoConfig.from_pretrained(name, trust_remote_code=config.trust_remote_code)
        custom = _CUSTOM_CLASSES.get(type(hf_config).__name__)
        if config.model_type == "custom" or config.custom_model_class is not None or custom is not None:
            cls = _resolve_class(config.custom_model_class or (custom or {}).get("model") or "AutoModel")
        else:
            cls = _auto_class(config, hf_config)
        if config.random_init:
            model = cls.from_config(hf_config) if hasattr(cls, "from_config") else cls(hf_config)
            if config.dtype is not None:
                model = model.to(config.dtype)
        else:
            model = cls.from_pretrained(name, config=hf_config, **kwargs)
    except HuggingFaceModelError:
        raise
    except Exception as ex:  # noqa: BLE001
        raise HuggingFaceModelError(name, f"The Hugging Face model '{name}' cannot be created: {ex}") from ex
    if config.device not in ("auto", "cpu") or (gangs is not None and getattr(gangs, "root", None) is not None):
        device = torch.device(config.device) if config.device not in ("auto",) else None
        if gangs is not None and getattr(gangs, "root", None) is not None:
            device = gangs.root.device  # type: ignore[attr-defined]
        if device is not None:
            model = model.to(device)
    if config.enable_gradient_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
        model.gradient_checkpointing_enable()
    return wrap_hg_model_if_causal_lm(model, hf_config)


class HgCausalLMAdapter(CausalLM):
    """Adapts a ``transformers`` causal LM to ``forward(seqs, seqs_layout, targets=...)``."""

    def __init__(self, hf_model: Module, hf_config: Any) -> None:
        max_len = int(getattr(hf_config, "max_position_embeddings", None) or getattr(hf_config, "n_positions", None)
                      or 2048)
        super().__init__(max_len)
        self._wrapped = hf_model
        self.hf_config = hf_config
        self.pad_idx = getattr(hf_config, "pad_token_id", None)

    @property
    def hf_model(self) -> Module:
        return self._wrapped

    def forward(self, seqs, seqs_layout, targets=None, *, state_bag=None, label_smoothing=0.0, target_mask=None,  # type: ignore[override]
                reduction="sum", return_logits=False):
        if state_bag is not None:
            raise NotImplementedError("Incremental decoding goes through `hf_model.generate()` for adapted models.")
        if seqs_layout.packed:
            raise ValueError("`HgCausalLMAdapter` does not support packed batches.")
        mask = None
        if seqs_layout.padded:
            mask = (seqs_layout.position_indices >= 0).to(torch.long)
        logits = self._wrapped(input_ids=seqs, attention_mask=mask).logits
        if targets is None:
            return logits
        loss = cross_entropy(logits, targets, self.pad_idx, label_smoothing=label_smoothing, target_mask=target_mask,
                             reduction=reduction)
        return (loss, logits) if return_logits else loss

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            wrapped = self.__dict__.get("_modules", {}).get("_wrapped")
            if wrapped is None:
                raise
            return getattr(wrapped, name)       # e.g. `generate`, `config`, `get_input_embeddings`


def wrap_hg_model_if_causal_lm(hf_model: Module, hf_config: Any) -> Module:
    name = type(hf_model).__name__
    if name.endswith("ForCausalLM") or name.endswith("LMHeadModel"):
        return HgCausalLMAdapter(hf_model, hf_config)
    return hf_model


# ------------------------------------------------------------------ simple API
def load_hg_model_simple(name: str | Path, *, model_type: str = "auto", device: str = "cpu",
                         dtype: DataType | None = None, trust_remote_code: bool = False, **kwargs: Any) -> Module:
    cfg = HuggingFaceModelConfig(hf_name=str(name), model_type=model_type, device=device, dtype=dtype,
                                 trust_remote_code=trust_remote_code, load_kwargs=kwargs or None)
    return create_hg_model(cfg)


def load_hg_tokenizer_simple(name: str | Path, *, trust_remote_code: bool = False, **kwargs: Any) -> Any:
    from fairseq2_b200.data.tokenizers.hg import HuggingFaceTokenizer

    return HuggingFaceTokenizer.from_pretrained(str(name), trust_remote_code=trust_remote_code, **kwargs) \
        if hasattr(HuggingFaceTokenizer, "from_pretrained") else HuggingFaceTokenizer(Path(name))


def load_causal_lm(name: str | Path, **kwargs: Any) -> Module:
    return load_hg_model_simple(name, model_type="causal_lm", **kwargs)


def load_seq2seq_lm(name: str | Path, **kwargs: Any) -> Module:
    return load_hg_model_simple(name, model_type="seq2seq_lm", **kwargs)
