"""Gemma 3n text decoder: AltUp (alternating updates over ``altup_num_inputs`` hidden streams), LAuReL low-rank
residuals, per-layer input embeddings, local/global attention with two RoPE bases, query/key/value RMS norms,
key/value sharing across the last layers, Gaussian top-k activation sparsity and final logit soft-capping
(cf. fairseq2 ``models/gemma3n/{altup,decoder_layer,decoder,frontend,model}.py``).

Tensor parallelism (``tp_gang`` of size > 1): the attention heads and the FFN inner dimension are split over the gang
(q/k/v and gate/up column-sharded, o and down row-sharded with an all-reduce of their outputs); everything that is
``model_dim`` wide -- embeddings, AltUp, LAuReL, per-layer inputs, norms, the output projection -- is replicated and
sees identical activations on every rank. The cut-off of the activation sparsity is a statistic over the whole
inner dimension: its two moments are summed over the gang.
"""
from __future__ import annotations

import math
from typing import Literal

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Module, ModuleList, Parameter

from fairseq2_b200.gang import Gang
from fairseq2_b200.models.gemma3n.config import Gemma3nConfig, is_global_layer, kv_source_layer
from fairseq2_b200.nn import BatchLayout
from fairseq2_b200.nn.functional import cross_entropy
from fairseq2_b200.nn.incremental_state import IncrementalState, IncrementalStateBag
from fairseq2_b200.nn.normalization import RMSNorm
from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, Projection, RowShardedLinear
from fairseq2_b200.ops.attention import varlen_attention
from fairseq2_b200.ops.tensor_parallel import reduce_both_ways, reduce_on_backward
from fairseq2_b200.typing import DataType, Device


def _rms(x: Tensor, eps: float) -> Tensor:
    """Scale-free RMS normalisation in fp32."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x)


def _column(tp: Gang | None, input_dim: int, output_dim: int, kw: dict) -> Projection:
    if tp is None or tp.size == 1:
        return Linear(input_dim, output_dim, bias=False, **kw)
    return ColumnShardedLinear(tp, input_dim, output_dim, False, gather_output=False, **kw)


def _row(tp: Gang | None, input_dim: int, output_dim: int, kw: dict) -> Projection:
    if tp is None or tp.size == 1:
        return Linear(input_dim, output_dim, bias=False, **kw)
    return RowShardedLinear(tp, input_dim, output_dim, False, scatter_input=False, **kw)


class AltUp(Module):
    """Predict-and-correct mixing of the hidden streams around a layer that only transforms the active one."""

    def __init__(self, cfg: Gemma3nConfig, device: Device | None, dtype: DataType | None) -> None:
        super().__init__()
        n, d = cfg.altup_num_inputs, cfg.model_dim
        kw = {"device": device, "dtype": dtype}
        self.n, self.active, self.clip = n, cfg.altup_active_idx, cfg.altup_coef_clip
        self.correct_output_scale = Parameter(torch.zeros(d, **kw))
        self.correction_coefs = Linear(n, n, bias=False, **kw)
        self.prediction_coefs = Linear(n, n * n, bias=False, **kw)
        self.modality_router = Linear(d, n, bias=False, **kw)
        self.router_norm = RMSNorm(d, bias=False, eps=cfg.rms_norm_eps, **kw)
        self.router_input_scale = 1.0 / d

    def _modalities(self, x: Tensor) -> Tensor:
        return torch.tanh(self.modality_router(self.router_norm(x) * self.router_input_scale).float()).type_as(x)

    def _clipped(self, w: Tensor) -> Tensor:
        return w.clamp(-self.clip, self.clip) if (self.training and self.clip is not None) else w

    def predict(self, streams: Tensor) -> Tensor:
        """``streams``: ``[n, ..., D]`` -> predictions of the same shape."""
        m = self._modalities(streams[self.active])                                    # [..., n]
        coefs = F.linear(m, self._clipped(self.prediction_coefs.weight))              # [..., n*n]
        coefs = coefs.reshape(*m.shape[:-1], self.n, self.n).transpose(-1, -2)
        x = streams.movedim(0, -1)                                                     # [..., D, n]
        pred = torch.matmul(x, coefs).movedim(-1, 0)
        return (pred + streams).contiguous().type_as(streams)

    def correct(self, predictions: Tensor, activated: Tensor) -> Tensor:
        m = self._modalities(activated)
        innovation = activated - predictions[self.active]
        coefs = F.linear(m, self._clipped(self.correction_coefs.weight)) + 1.0         # [..., n]
        coefs = coefs.movedim(-1, 0).unsqueeze(-1)
        return (innovation.unsqueeze(0) * coefs + predictions).contiguous().type_as(activated)

    def scale_corrected_output(self, x: Tensor) -> Tensor:
        return (x.type_as(self.correct_output_scale) * self.correct_output_scale).type_as(x)


class Laurel(Module):
    """``x + norm(right(left(x)))`` with a rank-``laurel_rank`` bottleneck."""

    def __init__(self, cfg: Gemma3nConfig, device: Device | None, dtype: DataType | None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.linear_left = Linear(cfg.model_dim, cfg.laurel_rank, bias=False, **kw)
        self.linear_right = Linear(cfg.laurel_rank, cfg.model_dim, bias=False, **kw)
        self.post_laurel_norm = RMSNorm(cfg.model_dim, bias=False, eps=cfg.rms_norm_eps, **kw)

    def forward(self, x: Tensor) -> Tensor:
        return x + self.post_laurel_norm(self.linear_right(self.linear_left(x)))


class Gemma3nFFN(Module):
    def __init__(self, cfg: Gemma3nConfig, sparsity: float, device: Device | None, dtype: DataType | None,
                 tp_gang: Gang | None = None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.tp = tp_gang if tp_gang is not None and tp_gang.size > 1 else None
        self.inner_dim = cfg.ffn_inner_dim
        self.gate_proj = _column(self.tp, cfg.model_dim, cfg.ffn_inner_dim, kw)
        self.up_proj = _column(self.tp, cfg.model_dim, cfg.ffn_inner_dim, kw)
        self.down_proj = _row(self.tp, cfg.ffn_inner_dim, cfg.model_dim, kw)
        self.sparsity = sparsity
        # standard-normal quantile of the target sparsity: entries below mean + z * std are zeroed
        self.std_multiplier = math.sqrt(2.0) * float(torch.erfinv(torch.tensor(2.0 * sparsity - 1.0))) if sparsity > 0 else 0.0

    def forward(self, x: Tensor) -> Tensor:
        gate = self.gate_proj(x)
        if self.sparsity > 0.0:
            if self.tp is None:
                mean = gate.mean(dim=-1, keepdim=True)
                std = gate.std(dim=-1, keepdim=True, unbiased=False)
            else:
                # this rank holds a slice of the inner dimension: first and second moment over all slices
                gf = gate.float()
                moments = reduce_both_ways(torch.stack([gf.sum(-1), gf.pow(2).sum(-1)], dim=-1), self.tp)
                mean = (moments[..., :1] / self.inner_dim)
                std = (moments[..., 1:] / self.inner_dim - mean.pow(2)).clamp_min(0.0).sqrt()
                mean, std = mean.type_as(gate), std.type_as(gate)
            gate = F.relu(gate - (mean + std * self.std_multiplier))
        return self.down_proj(F.gelu(gate, approximate="tanh") * self.up_proj(x))


def _rope_half(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Half-rotation RoPE: ``x`` ``[T, H, D]``, ``cos``/``sin`` ``[T, D]``."""
    d = x.shape[-1] // 2
    rot = torch.cat((-x[..., d:], x[..., :d]), dim=-1)
    return x * cos.unsqueeze(1) + rot * sin.unsqueeze(1)


class _KVState(IncrementalState):
    """Keys and values of one layer for all steps so far: ``[N, L, Hkv, D]``."""

    def __init__(self, k: Tensor, v: Tensor) -> None:
        self.k, self.v = k, v

    def append(self, k: Tensor, v: Tensor) -> None:
        self.k, self.v = torch.cat([self.k, k], dim=1), torch.cat([self.v, v], dim=1)

    def reorder(self, new_order: Tensor) -> None:
        self.k, self.v = self.k.index_select(0, new_order), self.v.index_select(0, new_order)

    def size_bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def capacity_bytes(self) -> int:
        return self.size_bytes()


class _AttnGeometry:
    """Flattened-token geometry of one forward call: where each sequence's queries and keys start and how long they
    are. Without a state bag keys = queries; with one, keys also cover the cached steps."""

    def __init__(self, q_begins: Tensor, q_lens: Tensor, max_q: int, batch: int | None, steps: int | None) -> None:
        self.q_begins, self.q_lens, self.max_q = q_begins, q_lens, max_q
        self.k_begins, self.k_lens, self.max_k = q_begins, q_lens, max_q
        self.batch, self.steps = batch, steps          # set in incremental mode: tokens are [batch, steps]

    def with_cache_len(self, total: int, device: torch.device) -> None:
        assert self.batch is not None
        self.k_begins = torch.arange(self.batch, device=device, dtype=torch.int32) * total
        self.k_lens = torch.full((self.batch,), total, device=device, dtype=torch.int32)
        self.max_k = total


class Gemma3nAttention(Module):
    def __init__(self, cfg: Gemma3nConfig, layer_idx: int, device: Device | None, dtype: DataType | None,
                 tp_gang: Gang | None = None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        H, Hkv, D = cfg.num_attn_heads, cfg.num_key_value_heads, cfg.head_dim
        tp = tp_gang if tp_gang is not None and tp_gang.size > 1 else None
        if tp is not None and (H % tp.size or Hkv % tp.size):
            raise ValueError(f"The tensor parallel size ({tp.size}) must divide the number of attention heads ({H}) "
                             f"and of key-value heads ({Hkv}).")
        shards = 1 if tp is None else tp.size
        # heads of this rank
        self.H, self.Hkv, self.D, self.eps = H // shards, Hkv // shards, D, cfg.rms_norm_eps
        self.is_global = is_global_layer(layer_idx, cfg.num_layers)
        self.window = None if self.is_global else cfg.sliding_window
        self.kv_source = kv_source_layer(layer_idx, cfg.num_layers, cfg.num_kv_shared_layers)
        self.q_proj = _column(tp, cfg.model_dim, H * D, kw)
        self.k_proj = _column(tp, cfg.model_dim, Hkv * D, kw)
        self.v_proj = _column(tp, cfg.model_dim, Hkv * D, kw)
        self.o_proj = _row(tp, H * D, cfg.model_dim, kw)
        self.q_norm = RMSNorm(D, bias=False, eps=cfg.rms_norm_eps, **kw)
        self.k_norm = RMSNorm(D, bias=False, eps=cfg.rms_norm_eps, **kw)
        self.tp = tp

    def _head_norm(self, norm: RMSNorm, x: Tensor) -> Tensor:
        """The per-head norms have one weight vector for all heads. With the heads split over ranks every rank
        only sees the gradient of its own heads: the weight enters through an identity whose backward pass sums
        over the gang, so the replicated weight gets the whole gradient on every rank."""
        if self.tp is None:
            return norm(x)
        return norm.apply_with(x, reduce_on_backward(norm.weight, self.tp), None)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor, geo: _AttnGeometry,
                shared_kv: dict[int, tuple[Tensor, Tensor]], layer_idx: int,
                state_bag: IncrementalStateBag | None = None) -> Tensor:
        """``x``: ``[T, D_model]`` (tokens of all sequences, flattened)."""
        T = x.shape[0]
        q = _rope_half(self._head_norm(self.q_norm, self.q_proj(x).view(T, self.H, self.D)), cos, sin)
        if self.kv_source is not None and self.kv_source in shared_kv:
            k, v = shared_kv[self.kv_source]
        else:
            k = _rope_half(self._head_norm(self.k_norm, self.k_proj(x).view(T, self.Hkv, self.D)), cos, sin)
            v = _rms(self.v_proj(x).view(T, self.Hkv, self.D), self.eps)
            if state_bag is not None:
                # keys/values of the earlier steps come from the cache; the new ones are appended
                kb, vb = k.view(geo.batch, geo.steps, self.Hkv, self.D), v.view(geo.batch, geo.steps, self.Hkv, self.D)
                state = state_bag.maybe_get_state(self, _KVState)
                if state is None:
                    state = _KVState(kb, vb)
                    state_bag.set_state(self, state)
                else:
                    state.append(kb, vb)
                k, v = state.k.reshape(-1, self.Hkv, self.D), state.v.reshape(-1, self.Hkv, self.D)
            shared_kv[layer_idx] = (k, v)
        if state_bag is not None:
            geo.with_cache_len(k.shape[0] // geo.batch, x.device)
        out = varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), geo.q_begins, geo.q_lens, geo.k_begins,
                               geo.k_lens, geo.max_q, geo.max_k, causal=True, scale=1.0, window=self.window)
        return self.o_proj(out.reshape(T, self.H * self.D))


class Gemma3nDecoderLayer(Module):
    def __init__(self, cfg: Gemma3nConfig, layer_idx: int, device: Device | None, dtype: DataType | None,
                 tp_gang: Gang | None = None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        d, p = cfg.model_dim, cfg.hidden_size_per_layer_input
        self.layer_idx, self.active, self.correct_scale = layer_idx, cfg.altup_active_idx, cfg.altup_correct_scale
        self.self_attn = Gemma3nAttention(cfg, layer_idx, device, dtype, tp_gang)
        self.mlp = Gemma3nFFN(cfg, cfg.activation_sparsity if layer_idx < cfg.num_sparse_layers else 0.0, device, dtype,
                              tp_gang)
        norm = lambda: RMSNorm(d, bias=False, eps=cfg.rms_norm_eps, **kw)  # noqa: E731
        self.input_layernorm, self.post_attention_layernorm = norm(), norm()
        self.pre_feedforward_layernorm, self.post_feedforward_layernorm = norm(), norm()
        self.altup = AltUp(cfg, device, dtype)
        self.laurel = Laurel(cfg, device, dtype)
        self.per_layer_input_gate = Linear(d, p, bias=False, **kw)
        self.per_layer_projection = Linear(p, d, bias=False, **kw)
        self.post_per_layer_input_norm = norm()

    def forward(self, streams: Tensor, per_layer_input: Tensor, cos: Tensor, sin: Tensor, geo: _AttnGeometry,
                shared_kv: dict[int, tuple[Tensor, Tensor]], state_bag: IncrementalStateBag | None = None) -> Tensor:
        predictions = self.altup.predict(streams)
        active = predictions[self.active]
        normed = self.input_layernorm(active)
        laurel = self.laurel(normed)
        attn = self.post_attention_layernorm(self.self_attn(normed, cos, sin, geo, shared_kv, self.layer_idx,
                                                            state_bag))
        attn_laurel = (active + attn + laurel) / math.sqrt(2.0)
        ffn = self.post_feedforward_layernorm(self.mlp(self.pre_feedforward_layernorm(attn_laurel)))
        corrected = self.altup.correct(predictions, attn_laurel + ffn)
        first = corrected[self.active].clone()
        if self.correct_scale:
            first = self.altup.scale_corrected_output(first)
        first = F.gelu(self.per_layer_input_gate(first), approximate="tanh") * per_layer_input
        first = self.post_per_layer_input_norm(self.per_layer_projection(first))
        return torch.cat([corrected[:1], corrected[1:] + first], dim=0)


class Gemma3nModel(Module):
    """Decoder-only LM with the ``TransformerLM`` calling convention: ``forward(seqs, layout, targets=None, ...)``."""

    def __init__(self, cfg: Gemma3nConfig, *, device: Device | None = None, dtype: DataType | None = None,
                 tp_gang: Gang | None = None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.cfg = cfg
        self.model_dim, self.pad_idx, self.max_seq_len = cfg.model_dim, cfg.pad_idx, cfg.max_seq_len
        d, L, p = cfg.model_dim, cfg.num_layers, cfg.hidden_size_per_layer_input
        self.embed_tokens = torch.nn.Embedding(cfg.vocab_size, d, padding_idx=cfg.pad_idx, **kw)
        self.embed_tokens_per_layer = torch.nn.Embedding(cfg.vocab_size_per_layer_input, L * p, padding_idx=cfg.pad_idx, **kw)
        self.per_layer_model_projection = Linear(d, L * p, bias=False, **kw)
        self.per_layer_projection_norm = RMSNorm(p, bias=False, eps=cfg.rms_norm_eps, **kw)
        self.altup_projections = ModuleList([Linear(d, d, bias=False, **kw) for _ in range(1, cfg.altup_num_inputs)])
        self.altup_unembed_projections = ModuleList([Linear(d, d, bias=False, **kw) for _ in range(1, cfg.altup_num_inputs)])
        self.layers = ModuleList([Gemma3nDecoderLayer(cfg, i, device, dtype, tp_gang) for i in range(L)])
        self.norm = RMSNorm(d, bias=False, eps=cfg.rms_norm_eps, **kw)
        self.lm_head: Linear | None = None if cfg.tied_embeddings else Linear(d, cfg.vocab_size, bias=False, **kw)
        self.audio_tower: Module | None = None
        self.embed_audio: Module | None = None
        if cfg.audio_config is not None:
            from fairseq2_b200.models.gemma3n.audio import Gemma3nAudioEncoder, Gemma3nMultimodalEmbedder

            self.audio_tower = Gemma3nAudioEncoder(cfg.audio_config, device=device, dtype=dtype)
            self.embed_audio = Gemma3nMultimodalEmbedder(cfg.audio_config, d, device=device, dtype=dtype)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for emb in (self.embed_tokens, self.embed_tokens_per_layer):
            if emb.weight.device.type != "meta":
                torch.nn.init.normal_(emb.weight, std=self.cfg.init_std)
                if emb.padding_idx is not None:
                    with torch.no_grad():
                        emb.weight[emb.padding_idx].zero_()

    # ------------------------------------------------------------------ pieces
    def _rope_tables(self, positions: Tensor, theta: float, dtype: torch.dtype) -> tuple[Tensor, Tensor]:
        D = self.cfg.head_dim
        inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=positions.device, dtype=torch.float32) / D))
        ang = positions.float().unsqueeze(-1) * inv
        emb = torch.cat((ang, ang), dim=-1)
        return emb.cos().to(dtype), emb.sin().to(dtype)

    def _per_layer_inputs(self, ids: Tensor, embeds: Tensor) -> Tensor:
        cfg = self.cfg
        L, p = cfg.num_layers, cfg.hidden_size_per_layer_input
        proj = (self.per_layer_model_projection(embeds) * cfg.model_dim ** -0.5).view(-1, L, p)
        proj = self.per_layer_projection_norm(proj)
        in_vocab = ids < cfg.vocab_size_per_layer_input
        tok = self.embed_tokens_per_layer(torch.where(in_vocab, ids, torch.zeros_like(ids))) * p ** 0.5
        tok = tok.view(-1, L, p) * in_vocab.view(-1, 1, 1)
        return (proj + tok.type_as(proj)) * (2.0 ** -0.5)

    @staticmethod
    def _match_magnitude(x: Tensor, target: Tensor) -> Tensor:
        mag = torch.sqrt(torch.clamp(x.pow(2).mean(-1, keepdim=True), min=1e-5))
        return x * target / mag

    def embed_inputs(self, ids: Tensor, audio_features: Tensor | None = None, audio_invalid: Tensor | None = None,
                     audio_token_idx: int | None = None, num_audio_tokens: int | None = None) -> Tensor:
        """Token embeddings ``[T, D]`` for flattened ids. Ids in the audio vocabulary range are embedded by the audio
        embedder; with ``audio_features`` (``[B, frames, mel_bins]``) the tower's soft tokens -- padded to
        ``num_audio_tokens`` per clip with the embedding of the last audio id -- replace, in order, the positions
        whose id is ``audio_token_idx``."""
        cfg = self.cfg
        x0 = self.embed_tokens(ids) * cfg.model_dim ** 0.5
        if self.embed_audio is None:
            return x0
        ac = cfg.audio_config
        assert ac is not None and self.audio_tower is not None
        hard = ids >= ac.vocab_offset
        last_id = ac.vocab_offset + ac.vocab_size - 1
        if bool(hard.any()):
            emb = self.embed_audio(input_ids=torch.where(hard, ids, torch.full_like(ids, last_id)))
            x0 = torch.where(hard.unsqueeze(-1), emb.to(x0.dtype), x0)
        if audio_features is not None:
            if audio_invalid is None:
                audio_invalid = torch.zeros(audio_features.shape[:2], dtype=torch.bool, device=audio_features.device)
            if audio_token_idx is None:
                raise ValueError("`audio_token_idx` (the placeholder id) must be given with `audio_features`.")
            enc, invalid = self.audio_tower(audio_features, audio_invalid)
            soft = self.embed_audio(inputs_embeds=enc)
            pad = self.embed_audio(input_ids=torch.full((1, 1), last_id, dtype=torch.long, device=ids.device))
            soft = torch.where(invalid.unsqueeze(-1), pad.to(soft.dtype), soft)
            if num_audio_tokens is not None and num_audio_tokens > soft.shape[1]:
                extra = pad.to(soft.dtype).expand(soft.shape[0], num_audio_tokens - soft.shape[1], -1)
                soft = torch.cat([soft, extra], dim=1)
            slots = ids == audio_token_idx
            if int(slots.sum()) != soft.shape[0] * soft.shape[1]:
                raise ValueError(f"The batch has {int(slots.sum())} audio placeholder tokens for "
                                 f"{soft.shape[0] * soft.shape[1]} audio soft tokens.")
            x0 = x0.masked_scatter(slots.unsqueeze(-1), soft.to(x0.dtype).reshape(-1, x0.shape[-1]))
        return x0

    def decode(self, seqs: Tensor, layout: BatchLayout, state_bag: IncrementalStateBag | None = None,
               inputs_embeds: Tensor | None = None) -> Tensor:
        """Token ids ``[N, S]`` or packed ``[T]`` -> final hidden states of the same leading shape. With a state bag
        ``seqs`` holds the next ``S`` steps of every sequence (unpadded) and attention also covers the cached steps."""
        cfg = self.cfg
        shape = seqs.shape
        ids = seqs.reshape(-1)
        T = ids.shape[0]
        if layout.packed:
            if state_bag is not None:
                raise ValueError("Incremental decoding needs an unpacked batch.")
            geo = _AttnGeometry(layout.seq_begin_indices_pt[:-1], layout.seq_lens_pt, layout.max_seq_len, None, None)
        else:
            S = shape[1]
            begins = (torch.arange(shape[0], device=ids.device, dtype=torch.int32) * S)
            geo = _AttnGeometry(begins, layout.seq_lens_pt, layout.max_seq_len, shape[0], S)
        positions = layout.position_indices.reshape(-1).clamp(min=0)
        if state_bag is not None:
            positions = positions + state_bag.step_nr
        x0 = inputs_embeds if inputs_embeds is not None else self.embed_inputs(ids)
        per_layer = self._per_layer_inputs(ids, x0)
        target = x0.pow(2).mean(-1, keepdim=True) ** 0.5
        streams = torch.stack([x0] + [self._match_magnitude(proj(x0), target) for proj in self.altup_projections])
        cos_l, sin_l = self._rope_tables(positions, cfg.rope_theta, x0.dtype)
        cos_g, sin_g = self._rope_tables(positions, cfg.rope_theta_global, x0.dtype)
        shared_kv: dict[int, tuple[Tensor, Tensor]] = {}
        for i, layer in enumerate(self.layers):
            cos, sin = (cos_g, sin_g) if layer.self_attn.is_global else (cos_l, sin_l)
            streams = layer(streams, per_layer[:, i], cos, sin, geo, shared_kv, state_bag)
        target = streams[0].pow(2).mean(-1, keepdim=True) ** 0.5
        outs = [streams[0]] + [self._match_magnitude(proj(streams[i + 1]), target)
                               for i, proj in enumerate(self.altup_unembed_projections)]
        h = self.norm(torch.stack(outs).mean(dim=0))
        del T
        return h.view(*shape, cfg.model_dim)

    def project(self, h: Tensor) -> Tensor:
        w = self.embed_tokens.weight if self.lm_head is None else self.lm_head.weight
        logits = F.linear(h, w)
        cap = self.cfg.final_logit_soft_cap
        if cap:
            logits = torch.tanh(logits.float() / cap).mul(cap).type_as(logits)
        return logits

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, targets: Tensor | None = None, *,
                state_bag: IncrementalStateBag | None = None,
                label_smoothing: float = 0.0, target_mask: Tensor | None = None,
                reduction: Literal["sum", "mean"] = "sum", return_logits: bool = False,
                audio_features: Tensor | None = None, audio_invalid: Tensor | None = None,
                audio_token_idx: int | None = None, num_audio_tokens: int | None = None):  # type: ignore[no-untyped-def]
        embeds = None
        if audio_features is not None:
            embeds = self.embed_inputs(seqs.reshape(-1), audio_features, audio_invalid, audio_token_idx, num_audio_tokens)
        logits = self.project(self.decode(seqs, seqs_layout, state_bag, embeds))
        if targets is None:
            return logits
        loss = cross_entropy(logits, targets, self.pad_idx, label_smoothing=label_smoothing, target_mask=target_mask,
                             reduction=reduction)
        return (loss, logits) if return_logits else loss
