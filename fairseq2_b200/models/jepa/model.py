"""JEPA vision encoder and its attentive-probe classifier (cf. fairseq2 ``models/jepa/config.py:22-158``,
``jepa/factory.py:49-283``, ``jepa/model.py``, ``jepa/classifier/model.py:30-229``, ``jepa/interop.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
from torch import Tensor
from torch.nn import GELU, Module, Parameter

from fairseq2_b200.models.llama.interop import convert_state_dict
from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache, IdentityBias
from fairseq2_b200.models.transformer.encoder import StandardTransformerEncoder, TransformerEncoder
from fairseq2_b200.models.transformer.encoder_layer import StandardTransformerEncoderLayer
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork, StandardFeedForwardNetwork
from fairseq2_b200.models.transformer.frontend import TransformerFrontend
from fairseq2_b200.models.transformer.multihead_attention import MultiheadAttention, StandardMultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.models.vit import Conv2dPatchFeatureExtractor, Conv3dPatchFeatureExtractor, StandardViTFrontend
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.normalization import LayerNorm, StandardLayerNorm
from fairseq2_b200.nn.position_encoder import Sinusoidal2dPositionEncoder, Sinusoidal3dPositionEncoder
from fairseq2_b200.nn.projection import Linear
from fairseq2_b200.nn.residual import DropPathResidualConnect
from fairseq2_b200.runtime.config_registry import ConfigRegistrar

JEPA_FAMILY = "jepa"
JEPA_CLASSIFIER_FAMILY = "jepa_classifier"


@dataclass(kw_only=True)
class JepaEncoderConfig:
    model_dim: int = 768
    num_input_channels: int = 3
    input_dims: tuple[int, ...] = (224, 224)
    """(height, width) for images, (depth, height, width) for videos."""
    patch_dims: tuple[int, ...] = (16, 16)
    num_encoder_layers: int = 12
    num_encoder_attn_heads: int = 12
    qkv_bias: bool = True
    attn_dropout_p: float = 0.0
    ffn_inner_dim_ratio: float = 4.0
    init_std: float = 0.02
    dropout_p: float = 0.0
    droppath_p: float = 0.0
    uniform_power: bool = False


@dataclass(kw_only=True)
class JepaConfig:
    encoder_config: JepaEncoderConfig = field(default_factory=JepaEncoderConfig)


@dataclass(kw_only=True)
class JepaClassifierConfig:
    encoder_config: JepaEncoderConfig = field(default_factory=JepaEncoderConfig)
    pool_depth: int = 1
    decoder_projection: bool = True
    num_queries: int = 1
    num_classes: int = 1000


arch = ConfigRegistrar(JepaConfig)
classifier_arch = ConfigRegistrar(JepaClassifierConfig)

_SIZES = {"tiny": (192, 12, 3, 4.0), "small": (384, 12, 6, 4.0), "base": (768, 12, 12, 4.0),
          "large": (1024, 24, 16, 4.0), "huge": (1280, 32, 16, 4.0), "giant": (1408, 40, 16, 48 / 11),
          "gigantic": (1664, 48, 16, 64 / 13)}


def _encoder_config(name: str) -> JepaEncoderConfig:
    d, n, h, r = _SIZES[name]
    return JepaEncoderConfig(model_dim=d, num_encoder_layers=n, num_encoder_attn_heads=h, ffn_inner_dim_ratio=r)


for _n in _SIZES:
    arch(_n)(lambda n=_n: JepaConfig(encoder_config=_encoder_config(n)))
for _n in ("base", "large", "huge"):
    classifier_arch(_n)(lambda n=_n: JepaClassifierConfig(encoder_config=_encoder_config(n)))


@arch("test")
def _jepa_test() -> JepaConfig:
    return JepaConfig(encoder_config=JepaEncoderConfig(model_dim=64, input_dims=(32, 32), patch_dims=(8, 8),
                                                       num_encoder_layers=2, num_encoder_attn_heads=4))


@classifier_arch("test")
def _jepa_classifier_test() -> JepaClassifierConfig:
    return JepaClassifierConfig(encoder_config=_jepa_test().encoder_config, num_classes=10, pool_depth=2)


def _trunc(w: Tensor, b: Tensor | None, std: float) -> None:
    torch.nn.init.trunc_normal_(w, std=std)
    if b is not None:
        torch.nn.init.zeros_(b)


class JepaModel(Module):
    def __init__(self, model_dim: int, encoder_frontend: TransformerFrontend, encoder: TransformerEncoder) -> None:
        super().__init__()
        self.model_dim, self.encoder_frontend, self.encoder = model_dim, encoder_frontend, encoder

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> tuple[Tensor, BatchLayout]:
        seqs, seqs_layout = self.encoder_frontend(seqs, seqs_layout)
        return self.encoder(seqs, seqs_layout), seqs_layout

    def extra_repr(self) -> str:
        return f"model_dim={self.model_dim}"


class JepaEncoderFactory:
    def __init__(self, config: JepaEncoderConfig) -> None:
        self._config = config

    def create_encoder_frontend(self) -> TransformerFrontend:
        c = self._config
        if len(c.input_dims) != len(c.patch_dims) or len(c.patch_dims) not in (2, 3):
            raise ValueError("`input_dims` and `patch_dims` must both have 2 or 3 entries.")
        std = c.init_std
        grid = tuple(i // p for i, p in zip(c.input_dims, c.patch_dims))
        if len(grid) == 3:
            fe: Module = Conv3dPatchFeatureExtractor(c.num_input_channels, c.model_dim, c.patch_dims,  # type: ignore[arg-type]
                                                     init_fn=lambda m: _trunc(m.weight, m.bias, std))
            pe: Any = Sinusoidal3dPositionEncoder(c.model_dim, grid, uniform_power=c.uniform_power)  # type: ignore[arg-type]
        else:
            fe = Conv2dPatchFeatureExtractor(c.num_input_channels, c.model_dim, c.patch_dims,  # type: ignore[arg-type]
                                             init_fn=lambda m: _trunc(m.weight, m.bias, std))
            pe = Sinusoidal2dPositionEncoder(c.model_dim, grid)  # type: ignore[arg-type]
        return StandardViTFrontend(fe, pe, dropout_p=c.dropout_p)  # type: ignore[arg-type]

    def create_encoder(self, num_layers: int | None = None) -> TransformerEncoder:
        c = self._config
        n = c.num_encoder_layers if num_layers is None else num_layers
        return StandardTransformerEncoder([self.create_encoder_layer(i) for i in range(n)], self.create_layer_norm())

    def _scaled_init(self, layer_idx: int):  # type: ignore[no-untyped-def]
        std = self._config.init_std

        def init(p: Linear) -> None:
            _trunc(p.weight, p.bias, std)
            with torch.no_grad():
                p.weight.div_((2.0 * (layer_idx + 1)) ** 0.5)

        return init

    def create_encoder_layer(self, layer_idx: int) -> StandardTransformerEncoderLayer:
        c = self._config
        drop = DropPathResidualConnect(c.droppath_p) if c.droppath_p > 0.0 else None
        drop2 = DropPathResidualConnect(c.droppath_p) if c.droppath_p > 0.0 else None
        return StandardTransformerEncoderLayer(self.create_self_attention(layer_idx), self.create_layer_norm(),
                                               self.create_ffn(layer_idx), self.create_layer_norm(),
                                               norm_order=TransformerNormOrder.PRE, self_attn_residual=drop,
                                               ffn_residual=drop2, dropout_p=c.dropout_p)

    def create_self_attention(self, layer_idx: int) -> MultiheadAttention:
        c = self._config
        std = c.init_std
        out = Linear(c.model_dim, c.model_dim, bias=True, init_fn=self._scaled_init(layer_idx))
        return StandardMultiheadAttention(c.model_dim, c.num_encoder_attn_heads,
                                          create_default_sdpa(IdentityBias(), dropout_p=c.attn_dropout_p),
                                          bias=c.qkv_bias, qkv_proj_init_fn=lambda p: _trunc(p.weight, p.bias, std),
                                          output_proj=out)

    def create_ffn(self, layer_idx: int) -> FeedForwardNetwork:
        c = self._config
        return StandardFeedForwardNetwork(c.model_dim, int(c.model_dim * c.ffn_inner_dim_ratio), bias=True,
                                          inner_activation=GELU(), proj_init_fn=self._scaled_init(layer_idx))

    def create_layer_norm(self) -> LayerNorm:
        return StandardLayerNorm(self._config.model_dim, bias=True, eps=1e-6)


def create_jepa_model(config: JepaConfig, gangs: object | None = None) -> JepaModel:
    f = JepaEncoderFactory(config.encoder_config)
    return JepaModel(config.encoder_config.model_dim, f.create_encoder_frontend(), f.create_encoder())


class CrossAttentionDecoderLayer(Module):
    """Pre-norm cross-attention (the norm is applied to the encoder output) followed by a pre-norm FFN."""

    def __init__(self, cross_attn_layer_norm: LayerNorm, cross_attn: MultiheadAttention, ffn_layer_norm: LayerNorm,
                 ffn: FeedForwardNetwork) -> None:
        super().__init__()
        self.cross_attn_layer_norm, self.cross_attn = cross_attn_layer_norm, cross_attn
        self.ffn_layer_norm, self.ffn = ffn_layer_norm, ffn

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, encoder_output: Tensor,
                encoder_output_layout: BatchLayout) -> Tensor:
        enc = self.cross_attn_layer_norm(encoder_output)
        seqs = seqs + self.cross_attn(seqs, seqs_layout, enc, encoder_output_layout, enc, AttentionBiasCache())
        return seqs + self.ffn(self.ffn_layer_norm(seqs))


class AttentivePooler(Module):
    """Learned query tokens cross-attend to the encoder output (optionally after extra encoder layers)."""

    def __init__(self, model_dim: int, decoder_layer: CrossAttentionDecoderLayer,
                 encoder: TransformerEncoder | None = None, *, num_queries: int = 1, init_std: float = 0.02) -> None:
        super().__init__()
        self.decoder_layer, self.encoder = decoder_layer, encoder
        self.query_tokens = Parameter(torch.empty((1, num_queries, model_dim)))
        self.init_std = init_std
        torch.nn.init.trunc_normal_(self.query_tokens, std=init_std)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> Tensor:
        if self.encoder is not None:
            seqs = self.encoder(seqs, seqs_layout)
        n = seqs.size(0)
        q = self.query_tokens.expand(n, -1, -1).contiguous()
        ql = BatchLayout(tuple(q.shape[:2]), [q.shape[1]] * n, device=q.device)
        return self.decoder_layer(q, ql, seqs, seqs_layout)

    def extra_repr(self) -> str:
        return f"num_queries={self.query_tokens.size(1)}"


class JepaClassifierModel(Module):
    def __init__(self, encoder_frontend: TransformerFrontend, encoder: TransformerEncoder, pooler: AttentivePooler,
                 head: Linear) -> None:
        super().__init__()
        self.model_dim = encoder.layers[0].self_attn.model_dim if hasattr(encoder, "layers") else 0  # type: ignore[index,union-attr]
        self.encoder_frontend, self.encoder, self.pooler, self.head = encoder_frontend, encoder, pooler, head

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout) -> Tensor:
        seqs, layout = self.encoder_frontend(seqs, seqs_layout)
        seqs = self.encoder(seqs, layout)
        pooled = self.pooler(seqs, layout).squeeze(1)
        return self.head(pooled)


def create_jepa_classifier_model(config: JepaClassifierConfig, gangs: object | None = None) -> JepaClassifierModel:
    c, e = config, config.encoder_config
    f = JepaEncoderFactory(e)
    std = e.init_std
    out = Linear(e.model_dim, e.model_dim, bias=True, init_fn=lambda p: _trunc(p.weight, p.bias, std)) \
        if c.decoder_projection else None
    cross = StandardMultiheadAttention(e.model_dim, e.num_encoder_attn_heads, create_default_sdpa(IdentityBias()),
                                       bias=e.qkv_bias, qkv_proj_init_fn=lambda p: _trunc(p.weight, p.bias, std),
                                       output_proj=out)
    ffn = StandardFeedForwardNetwork(e.model_dim, int(e.model_dim * e.ffn_inner_dim_ratio), bias=True,
                                     inner_activation=GELU(), proj_init_fn=lambda p: _trunc(p.weight, p.bias, std))
    layer = CrossAttentionDecoderLayer(f.create_layer_norm(), cross, f.create_layer_norm(), ffn)
    extra = f.create_encoder(c.pool_depth - 1) if c.pool_depth > 1 else None
    pooler = AttentivePooler(e.model_dim, layer, extra, num_queries=c.num_queries, init_std=std)
    head = Linear(e.model_dim, c.num_classes, bias=True, init_fn=lambda p: _trunc(p.weight, p.bias, std))
    return JepaClassifierModel(f.create_encoder_frontend(), f.create_encoder(), pooler, head)


_JEPA_KEY_MAP = {
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.attn\.q_proj\.": r"encoder.layers.\2.self_attn.q_proj.",
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.attn\.k_proj\.": r"encoder.layers.\2.self_attn.k_proj.",
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.attn\.v_proj\.": r"encoder.layers.\2.self_attn.v_proj.",
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.attn\.proj\.": r"encoder.layers.\2.self_attn.output_proj.",
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.norm1\.": r"encoder.layers.\2.self_attn_layer_norm.",
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.mlp\.fc1\.": r"encoder.layers.\2.ffn.inner_proj.",
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.mlp\.fc2\.": r"encoder.layers.\2.ffn.output_proj.",
    r"^(module\.)?backbone\.blocks\.([0-9]+)\.norm2\.": r"encoder.layers.\2.ffn_layer_norm.",
    r"^(module\.)?backbone\.norm\.": r"encoder.layer_norm.",
    r"^(module\.)?backbone\.patch_embed\.proj\.": r"encoder_frontend.patch_feature_extractor.conv.",
}


def convert_jepa_state_dict(sd: dict[str, Any], config: JepaConfig) -> dict[str, Any]:
    """Original JEPA checkpoints keep the encoder under ``encoder``/``target_encoder`` with fused ``qkv`` weights."""
    for key in ("target_encoder", "encoder"):
        if key in sd and isinstance(sd[key], dict):
            sd = sd[key]
            break
    if not any("backbone.blocks" in k for k in sd):
        return dict(sd)
    split: dict[str, Any] = {}
    for k, v in sd.items():
        if k.endswith("pos_embed"):
            continue                                   # positions are a fixed sinusoidal table here
        if ".attn.qkv." in k:
            q, kk, vv = v.chunk(3, dim=0)
            for name, t in (("q_proj", q), ("k_proj", kk), ("v_proj", vv)):
                split[k.replace(".attn.qkv.", f".attn.{name}.")] = t
        else:
            split[k] = v
    return convert_state_dict(split, _JEPA_KEY_MAP)
