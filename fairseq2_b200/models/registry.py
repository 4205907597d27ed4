"""Registers the built-in model families."""
from __future__ import annotations

from torch.nn import Module

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
    layerwise_ac_applier=apply_layerwise_ac, hg_exporter=export_llama_to_hg, supports_sequence_parallel=True))


def _register_lm_families() -> None:
    from fairseq2_b200.models.mistral import (MISTRAL_FAMILY, MistralConfig, convert_mistral_state_dict,
                                              create_mistral_model, export_mistral_to_hg)
    from fairseq2_b200.models.olmo import (OLMO_FAMILY, OLMOConfig, convert_olmo_state_dict, create_olmo_model,
                                           export_olmo_to_hg)
    from fairseq2_b200.models.qwen import (QWEN_FAMILY, QwenConfig, convert_qwen_state_dict, create_qwen_model,
                                           export_qwen_to_hg)

    for name, cfg, factory, conv, exp in (
            (MISTRAL_FAMILY, MistralConfig, create_mistral_model, convert_mistral_state_dict, export_mistral_to_hg),
            (QWEN_FAMILY, QwenConfig, create_qwen_model, convert_qwen_state_dict, export_qwen_to_hg),
            (OLMO_FAMILY, OLMOConfig, create_olmo_model, convert_olmo_state_dict, export_olmo_to_hg)):
        register_model_family(ModelFamily(
            name=name, kls=TransformerLM, config_kls=cfg, factory=factory, state_dict_converter=conv,
            fsdp_wrap_policy=layerwise_wrap_policy, layerwise_ac_applier=apply_layerwise_ac, hg_exporter=exp))

    from fairseq2_b200.models.llama4 import LLAMA4_FAMILY, Llama4Config, convert_llama4_state_dict, create_llama4_model

    register_model_family(ModelFamily(
        name=LLAMA4_FAMILY, kls=TransformerLM, config_kls=Llama4Config, factory=create_llama4_model,
        state_dict_converter=convert_llama4_state_dict, fsdp_wrap_policy=layerwise_wrap_policy,
        layerwise_ac_applier=apply_layerwise_ac))


    from fairseq2_b200.models.moe_lm import MOE_LM_FAMILY, MoELMConfig, MoETransformerLM, create_moe_lm_model

    register_model_family(ModelFamily(
        name=MOE_LM_FAMILY, kls=MoETransformerLM, config_kls=MoELMConfig, factory=create_moe_lm_model,
        fsdp_wrap_policy=layerwise_wrap_policy, layerwise_ac_applier=apply_layerwise_ac))

    from fairseq2_b200.models.gemma3n import (GEMMA3N_FAMILY, Gemma3nConfig, Gemma3nModel, convert_gemma3n_state_dict,
                                              create_gemma3n_model, export_gemma3n_to_hg, gemma3n_wrap_policy)

    register_model_family(ModelFamily(
        name=GEMMA3N_FAMILY, kls=Gemma3nModel, config_kls=Gemma3nConfig, factory=create_gemma3n_model,
        state_dict_converter=convert_gemma3n_state_dict, fsdp_wrap_policy=gemma3n_wrap_policy,
        hg_exporter=export_gemma3n_to_hg))


_register_lm_families()


def _encoder_wrap_policy(module):  # type: ignore[no-untyped-def]
    """One FSDP unit per encoder layer (speech encoders keep the front end in the root unit)."""
    enc = getattr(module, "encoder", None)
    return list(enc.layers) if enc is not None and hasattr(enc, "layers") else []


def _register_speech_families() -> None:
    from fairseq2_b200.models.wav2vec2 import (WAV2VEC2_FAMILY, Wav2Vec2Config, Wav2Vec2Model,
                                               convert_wav2vec2_asr_state_dict, convert_wav2vec2_state_dict,
                                               create_wav2vec2_model)
    from fairseq2_b200.models.wav2vec2.asr import (WAV2VEC2_ASR_FAMILY, Wav2Vec2AsrConfig, Wav2Vec2AsrModel,
                                                   create_wav2vec2_asr_model)

    register_model_family(ModelFamily(
        name=WAV2VEC2_FAMILY, kls=Wav2Vec2Model, config_kls=Wav2Vec2Config, factory=create_wav2vec2_model,
        state_dict_converter=convert_wav2vec2_state_dict, fsdp_wrap_policy=_encoder_wrap_policy, supports_meta=False))
    register_model_family(ModelFamily(
        name=WAV2VEC2_ASR_FAMILY, kls=Wav2Vec2AsrModel, config_kls=Wav2Vec2AsrConfig,
        factory=create_wav2vec2_asr_model, state_dict_converter=convert_wav2vec2_asr_state_dict,
        fsdp_wrap_policy=_encoder_wrap_policy, supports_meta=False))

    from fairseq2_b200.models.nllb import NLLB_FAMILY, NllbConfig, convert_nllb_state_dict, create_nllb_model
    from fairseq2_b200.models.s2t_transformer import (S2T_CONFORMER_FAMILY, S2T_TRANSFORMER_FAMILY, S2TConformerConfig,
                                                      S2TTransformerConfig, convert_s2t_state_dict,
                                                      create_s2t_conformer_model, create_s2t_transformer_model)
    from fairseq2_b200.models.transformer.model import TransformerModel
    from fairseq2_b200.models.w2vbert import W2VBERT_FAMILY, W2VBertConfig, W2VBertModel, create_w2vbert_model

    def enc_dec_policy(module):  # type: ignore[no-untyped-def]
        return list(module.encoder.layers) + list(module.decoder.layers)

    register_model_family(ModelFamily(
        name=NLLB_FAMILY, kls=TransformerModel, config_kls=NllbConfig, factory=create_nllb_model,
        state_dict_converter=convert_nllb_state_dict, fsdp_wrap_policy=enc_dec_policy, supports_meta=False))
    register_model_family(ModelFamily(
        name=S2T_TRANSFORMER_FAMILY, kls=TransformerModel, config_kls=S2TTransformerConfig,
        factory=create_s2t_transformer_model, state_dict_converter=convert_s2t_state_dict,
        fsdp_wrap_policy=enc_dec_policy, supports_meta=False))
    register_model_family(ModelFamily(
        name=S2T_CONFORMER_FAMILY, kls=TransformerModel, config_kls=S2TConformerConfig,
        factory=create_s2t_conformer_model, state_dict_converter=convert_s2t_state_dict,
        fsdp_wrap_policy=enc_dec_policy, supports_meta=False))
    register_model_family(ModelFamily(
        name=W2VBERT_FAMILY, kls=W2VBertModel, config_kls=W2VBertConfig, factory=create_w2vbert_model,
        fsdp_wrap_policy=lambda m: list(m.w2v2_model.encoder.layers), supports_meta=False))


_register_speech_families()


def _register_vision_families() -> None:
    from fairseq2_b200.models.jepa import (JEPA_CLASSIFIER_FAMILY, JEPA_FAMILY, JepaClassifierConfig,
                                           JepaClassifierModel, JepaConfig, JepaModel, convert_jepa_state_dict,
                                           create_jepa_classifier_model, create_jepa_model)

    register_model_family(ModelFamily(
        name=JEPA_FAMILY, kls=JepaModel, config_kls=JepaConfig, factory=create_jepa_model,
        state_dict_converter=convert_jepa_state_dict, fsdp_wrap_policy=_encoder_wrap_policy, supports_meta=False))
    register_model_family(ModelFamily(
        name=JEPA_CLASSIFIER_FAMILY, kls=JepaClassifierModel, config_kls=JepaClassifierConfig,
        factory=create_jepa_classifier_model, fsdp_wrap_policy=_encoder_wrap_policy, supports_meta=False))


_register_vision_families()


def _register_hg_family() -> None:
    from fairseq2_b200.models.hg import HG_FAMILY, HuggingFaceModelConfig, create_hg_model

    def hg_policy(module):  # type: ignore[no-untyped-def]
        """FSDP units: the repeated decoder/encoder blocks of the wrapped model (largest ModuleList)."""
        import torch

        best = []
        for m in module.modules():
            if isinstance(m, torch.nn.ModuleList) and len(m) > len(best):
                best = list(m)
        return best

    register_model_family(ModelFamily(
        name=HG_FAMILY, kls=Module, config_kls=HuggingFaceModelConfig, factory=create_hg_model,
        fsdp_wrap_policy=hg_policy, supports_meta=False))


_register_hg_family()
