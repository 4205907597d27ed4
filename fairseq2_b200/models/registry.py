"""Registers the built-in model families."""
from __future__ import annotations

from fairseq2_b200.models.family import ModelFamily, register_model_family
from fairseq2_b200.models.llama.config import LLAMA_FAMILY, LLaMAConfig
from fairseq2_b200.models.llama.factory import create_llama_model
from fairseq2_b200.models.llama.interop import convert_llama_state_dict, export_llama_to_hg
from fairseq2_b200.models.transformer_lm import TransformerLM
from fairseq2_b200.models.utils_ac import apply_layerwise_ac
from fairseq2_b200.parallel.fsdp import layerwise_wrap_policy

register_model_family(ModelFamily(
    name=LLAMA_FAMILY, kls=TransformerLM, config_kls=LLaMAConfig, factory=create_llama_model,
    state_dict_converter=convert_llama_state_dict, fsdp_wrap_policy=layerwise_wrap_policy,
    layerwise_ac_applier=apply_layerwise_ac, hg_exporter=export_llama_to_hg))
