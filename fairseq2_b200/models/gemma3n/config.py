"""Gemma 3n configuration: text decoder and audio tower (cf. fairseq2 ``models/gemma3n/config.py:27-274``)."""
from __future__ import annotations

from dataclasses import dataclass

from fairseq2_b200.runtime.config_registry import ConfigRegistrar

GEMMA3N_FAMILY = "gemma3n"


@dataclass(kw_only=True)
class Gemma3nAudioConfig:
    """Audio tower (Universal-Speech-Model conformer); defaults are the E2B/E4B tower
    (cf. fairseq2 ``models/gemma3n/config.py:27-92``)."""

    vocab_size: int = 128
    vocab_offset: int = 262_272
    input_feat_size: int = 128
    hidden_size: int = 1536
    rms_norm_eps: float = 1e-6
    gradient_clipping: float = 1e10
    conf_num_hidden_layers: int = 12
    conf_num_attention_heads: int = 8
    conf_conv_kernel_size: int = 5
    conf_attention_chunk_size: int = 12
    conf_attention_context_left: int = 13
    conf_attention_context_right: int = 0
    conf_attention_logit_cap: float = 50.0
    conf_reduction_factor: int = 4
    conf_residual_weight: float = 0.5
    sscp_conv_channel_size: tuple[int, int] = (128, 32)
    sscp_conv_group_norm_eps: float = 1e-3
    sscp_conv_kernel_size: tuple[tuple[int, int], tuple[int, int]] = ((3, 3), (3, 3))
    sscp_conv_stride_size: tuple[tuple[int, int], tuple[int, int]] = ((2, 2), (2, 2))


@dataclass(kw_only=True)
class Gemma3nConfig:
    model_dim: int = 2048
    max_seq_len: int = 32_768
    vocab_size: int = 262_400
    pad_idx: int | None = 0
    tied_embeddings: bool = True
    num_layers: int = 35
    num_attn_heads: int = 8
    num_key_value_heads: int = 2
    head_dim: int = 256
    ffn_inner_dim: int = 16_384
    sliding_window: int = 512
    """Window of the local layers; every 5th layer and the last one attend globally."""
    rope_theta: float = 10_000.0
    """RoPE base of the local layers."""
    rope_theta_global: float = 1_000_000.0
    final_logit_soft_cap: float | None = 30.0
    num_kv_shared_layers: int = 15
    """The last this-many layers reuse the keys/values of the last earlier layer of the same kind."""
    activation_sparsity: float = 0.95
    """Target sparsity of the FFN gate in the first ``num_sparse_layers`` layers (Gaussian top-k)."""
    num_sparse_layers: int = 10
    laurel_rank: int = 64
    altup_num_inputs: int = 4
    altup_active_idx: int = 0
    altup_coef_clip: float | None = 120.0
    altup_correct_scale: bool = True
    vocab_size_per_layer_input: int = 262_144
    hidden_size_per_layer_input: int = 256
    rms_norm_eps: float = 1e-6
    init_std: float = 0.02
    audio_config: Gemma3nAudioConfig | None = None
    """When set, the model carries the audio tower and its embedder; ``forward`` then accepts mel features."""


def is_global_layer(layer_idx: int, num_layers: int) -> bool:
    """4 local : 1 global; layers 4, 9, 14, ... are global."""
    return (layer_idx + 1) % 5 == 0


def kv_source_layer(layer_idx: int, num_layers: int, num_kv_shared_layers: int) -> int | None:
    """For a layer among the last ``num_kv_shared_layers``: the index of the last earlier, non-sharing layer of the
    same kind (local/global), whose keys and values it reuses. ``None`` for layers that compute their own."""
    first_shared = num_layers - num_kv_shared_layers
    if num_kv_shared_layers <= 0 or layer_idx < first_shared:
        return None
    kind = is_global_layer(layer_idx, num_layers)
    for idx in range(first_shared - 1, -1, -1):
        if is_global_layer(idx, num_layers) == kind:
            return idx
    return None


arch = ConfigRegistrar(Gemma3nConfig)


@arch("e4b")
def gemma3n_e4b() -> Gemma3nConfig:
    return Gemma3nConfig(audio_config=Gemma3nAudioConfig())


@arch("e2b")
def gemma3n_e2b() -> Gemma3nConfig:
    return Gemma3nConfig(num_layers=30, ffn_inner_dim=8192, num_kv_shared_layers=10, audio_config=Gemma3nAudioConfig())


@arch("e4b_text")
def gemma3n_e4b_text() -> Gemma3nConfig:
    return Gemma3nConfig()


@arch("tiny")
def gemma3n_tiny() -> Gemma3nConfig:
    return Gemma3nConfig(model_dim=64, max_seq_len=128, vocab_size=320, num_layers=6, num_attn_heads=4,
                         num_key_value_heads=2, head_dim=16, ffn_inner_dim=128, sliding_window=8, num_kv_shared_layers=0,
                         num_sparse_layers=2, laurel_rank=8, vocab_size_per_layer_input=320,
                         hidden_size_per_layer_input=16)
