"""Builds mixture-of-experts language models (see ``config.py``)."""
from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from fairseq2_b200.gang import Gangs, get_current_gangs
from fairseq2_b200.models.moe_lm.config import MoELMConfig
from fairseq2_b200.models.transformer.attention_bias import CausalAttentionBias
from fairseq2_b200.models.transformer.experts import MoE
from fairseq2_b200.models.transformer.frontend import TransformerEmbeddingFrontend
from fairseq2_b200.models.transformer.multihead_attention import StandardMultiheadAttention
from fairseq2_b200.models.transformer.norm_order import TransformerNormOrder
from fairseq2_b200.models.transformer.sdpa import create_default_sdpa
from fairseq2_b200.models.transformer_lm import (StandardTransformerLMDecoder, StandardTransformerLMDecoderLayer,
                                                 TransformerLM)
from fairseq2_b200.nn.embedding import StandardEmbedding
from fairseq2_b200.nn.normalization import RMSNorm
from fairseq2_b200.nn.position_encoder import RotaryEncoder
from fairseq2_b200.nn.projection import Linear


class MoETransformerLM(TransformerLM):
    """Decoder-only LM whose training loss includes the routers' load-balancing losses: with ``targets`` the
    returned (sum-reduced) loss is ``cross_entropy + aux_loss_coef * num_targets * mean_over_layers(aux)``, so that
    after the trainer's division by the number of targets the auxiliary term has weight ``aux_loss_coef``."""

    aux_loss_coef: float = 0.0

    def forward(self, seqs, seqs_layout, targets=None, *, state_bag=None, label_smoothing=0.0, target_mask=None,  # type: ignore[override]
                reduction="sum", return_logits=False):
        out = super().forward(seqs, seqs_layout, targets, state_bag=state_bag, label_smoothing=label_smoothing,
                              target_mask=target_mask, reduction=reduction, return_logits=return_logits)
        if targets is None or self.aux_loss_coef == 0.0 or not self.training:
            return out
        aux = [layer.ffn.last_aux_loss for layer in self.decoder.layers
               if isinstance(getattr(layer, "ffn", None), MoE) and layer.ffn.last_aux_loss is not None]
        if not aux:
            return out
        term = torch.stack(aux).mean() * self.aux_loss_coef
        if reduction == "sum":
            n = target_mask.sum() if target_mask is not None else torch.tensor(float(targets.numel()))
            term = term * n.to(term.device, term.dtype)
        if isinstance(out, tuple):
            return (out[0] + term.to(out[0].dtype), *out[1:])
        return out + term.to(out.dtype)


def create_moe_lm_model(config: MoELMConfig, gangs: Gangs | None = None, *, ep: Any | None = None) -> MoETransformerLM:
    """``ep``: an ``ops.moe_ep.ExpertParallelExchange`` shared by all layers; with it every rank builds only its own
    ``num_experts / world`` experts."""
    return MoELMFactory(config, gangs, ep=ep).create_model()


class MoELMFactory:
    def __init__(self, config: MoELMConfig, gangs: Gangs | None = None, *, ep: Any | None = None) -> None:
        self._config = config
        self._gangs = gangs if gangs is not None else get_current_gangs()
        self._ep = ep if ep is not None else self._maybe_create_exchange()

    def _maybe_create_exchange(self) -> Any | None:
        """The expert-parallel exchange over the data-parallel gang when ``config.expert_parallel`` asks for it."""
        c, dp = self._config, self._gangs.dp
        if not c.expert_parallel or dp.size == 1:
            return None
        from fairseq2_b200.error import NotSupportedError
        from fairseq2_b200.parallel.symm import SymmetricArena, symmetric_memory_available

        if self._gangs.tp.size > 1:
            raise NotSupportedError("Expert parallelism cannot be combined with tensor parallelism.")
        if c.num_experts % dp.size:
            raise NotSupportedError(f"`num_experts` ({c.num_experts}) must be a multiple of the data-parallel size "
                                    f"({dp.size}) for expert parallelism.")
        if not symmetric_memory_available(dp):
            raise NotSupportedError("Expert parallelism needs 2 to 8 CUDA ranks with peer access (one NVSwitch domain).")
        from fairseq2_b200.ops.moe_ep import ExpertParallelExchange

        rows = c.ep_max_tokens * c.top_k
        cap = int(c.ep_capacity_factor * rows)
        per_box = (cap + 128 * (c.num_experts // dp.size + 2)) * c.model_dim * 2
        with torch.device(dp.device):                       # the model itself may be under construction on "meta"
            arena = SymmetricArena(dp.base_gang(), 2 * per_box + (8 << 20), wait_limit_s=120.0)  # type: ignore[arg-type]
            return ExpertParallelExchange(arena, c.num_experts, c.model_dim, max_tokens=c.ep_max_tokens,
                                          top_k=c.top_k, capacity=cap)

    def _init(self, p: Linear) -> None:
        std = self._config.init_std or p.weight.shape[1] ** -0.5
        torch.nn.init.trunc_normal_(p.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
        if p.bias is not None:
            torch.nn.init.zeros_(p.bias)

    def create_model(self) -> MoETransformerLM:
        c = self._config

        def init_embed(e: StandardEmbedding) -> None:
            std = c.init_std or c.model_dim ** -0.5
            torch.nn.init.trunc_normal_(e.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

        embed = StandardEmbedding(c.vocab_size, c.model_dim, c.pad_idx, init_fn=init_embed)
        frontend = TransformerEmbeddingFrontend(c.model_dim, embed, pos_encoder=None, no_scale=True,
                                                dropout_p=c.dropout_p)
        pe = RotaryEncoder(c.head_dim, c.max_seq_len, theta=c.rope_theta)
        layers = [self.create_layer(i, pe) for i in range(c.num_layers)]
        decoder = StandardTransformerLMDecoder(layers, RMSNorm(c.model_dim, bias=False))
        final = Linear(c.model_dim, c.vocab_size, bias=False, init_fn=self._init)
        model = MoETransformerLM(c.model_dim, frontend, decoder, final, c.pad_idx, c.max_seq_len)
        model.aux_loss_coef = c.aux_loss_coef
        if self._ep is not None:
            from fairseq2_b200.models.transformer.experts import GroupedExpertNetwork

            # each rank's experts are its own: the sharded data-parallel wrapper keeps them as rank-local units
            model.fsdp_local_module_filter = lambda m: isinstance(m, GroupedExpertNetwork)
            model.expert_parallel_exchange = self._ep
        return model

    def create_layer(self, idx: int, pe: RotaryEncoder) -> StandardTransformerLMDecoderLayer:
        c = self._config
        attn = StandardMultiheadAttention(c.model_dim, c.num_attn_heads, create_default_sdpa(CausalAttentionBias()),
                                          head_dim=c.head_dim, num_key_value_heads=c.num_key_value_heads,
                                          qkv_proj_init_fn=self._init, pos_encoder=pe, output_proj_init_fn=self._init,
                                          bias=False)
        ffn = MoE(c.model_dim, c.expert_inner_dim, False, c.num_experts, 1.0, c.top_k, inner_dim_scale=1.0,
                  auto_scale=False, ep=self._ep, softmax_gate=True, aux_loss=c.aux_loss_coef > 0.0,
                  router_init_std=c.router_init_std)
        return StandardTransformerLMDecoderLayer(attn, RMSNorm(c.model_dim, bias=False), ffn,
                                                 RMSNorm(c.model_dim, bias=False), norm_order=TransformerNormOrder.PRE,
                                                 dropout_p=c.dropout_p)
