"""OLMo-2 / OLMo-3 configuration (cf. fairseq2 ``models/olmo/config.py:20-330``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

from fairseq2_b200.runtime.config_registry import ConfigRegistrar

OLMO_FAMILY = "olmo"


@dataclass(kw_only=True)
class YaRNScaleConfig:
    """YaRN context extension (8K -> 65K in OLMo-3)."""

    scale_factor: float = 8.0
    original_max_seq_len: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    truncate: bool = True


@dataclass(kw_only=True)
class OLMOConfig:
    model_dim: int = 2048
    max_seq_len: int = 4096
    vocab_size: int = 100_352
    pad_idx: int = 100_277
    bos_token_id: int | None = None
    eos_token_id: int = 100_257
    tied_embeddings: bool = False
    num_layers: int = 16
    num_attn_heads: int = 16
    num_key_value_heads: int = 16
    ffn_inner_dim: int = 8192
    """The final FFN width (HF ``intermediate_size``); no scaling or rounding is applied."""
    rms_norm_eps: float = 1e-6
    rope_theta: float = 500_000.0
    dropout_p: float = 0.0
    init_std: float | None = None
    init_std_scale: Literal["none", "layer", "stack"] = "layer"
    shard_embed_dim: bool = True
    sliding_window: int | None = None
    """If set, three of every four layers attend within this window; every fourth and the last attend globally."""
    layer_types: list[Literal["sliding_attention", "full_attention"]] | None = None
    yarn_scale_config: YaRNScaleConfig | None = None

    def resolved_layer_types(self) -> list[str]:
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_layers:
                raise ValueError(f"`layer_types` must have {self.num_layers} entries, but has {len(self.layer_types)}.")
            return list(self.layer_types)
        if self.sliding_window is None:
            return ["full_attention"] * self.num_layers
        return ["full_attention" if (i == self.num_layers - 1 or (i + 1) % 4 == 0) else "sliding_attention"
                for i in range(self.num_layers)]


arch = ConfigRegistrar(OLMOConfig)


def _olmo3(c: OLMOConfig) -> OLMOConfig:
    c.vocab_size = 100_278
    c.max_seq_len = 65_536
    c.sliding_window = 4096
    c.yarn_scale_config = YaRNScaleConfig()
    return c


@arch("olmo2_1b")
def olmo2_1b() -> OLMOConfig:
    return OLMOConfig()


@arch("olmo2_7b")
def olmo2_7b() -> OLMOConfig:
    return OLMOConfig(model_dim=4096, ffn_inner_dim=11008, num_layers=32, num_attn_heads=32, num_key_value_heads=32)


@arch("olmo2_13b")
def olmo2_13b() -> OLMOConfig:
    return OLMOConfig(model_dim=5120, ffn_inner_dim=13824, num_layers=40, num_attn_heads=40, num_key_value_heads=40)


@arch("olmo2_32b")
def olmo2_32b() -> OLMOConfig:
    return OLMOConfig(model_dim=5120, ffn_inner_dim=13824, num_layers=64, num_attn_heads=40, num_key_value_heads=8)


@arch("olmo3_7b")
def olmo3_7b() -> OLMOConfig:
    return _olmo3(olmo2_7b())


@arch("olmo3_32b")
def olmo3_32b() -> OLMOConfig:
    return _olmo3(OLMOConfig(model_dim=5120, ffn_inner_dim=27648, num_layers=64, num_attn_heads=40,
                             num_key_value_heads=8))


@arch("tiny")
def olmo_tiny() -> OLMOConfig:
    return OLMOConfig(model_dim=128, max_seq_len=256, vocab_size=512, pad_idx=0, num_layers=4, num_attn_heads=2,
                      num_key_value_heads=2, ffn_inner_dim=256, sliding_window=16,
                      yarn_scale_config=YaRNScaleConfig(scale_factor=4.0, original_max_seq_len=64))
