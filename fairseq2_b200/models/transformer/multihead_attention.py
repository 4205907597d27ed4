"""Multi-head attention with GQA, RoPE, q/k norms and KV caches
(cf. fairseq2 ``models/transformer/multihead_attention.py:150-965``).

Training / prefill fast path: when q, k and v projection weights sit back to
back in one storage (the FSDP flat buffers lay them out that way) a single GEMM
produces the merged ``[T, H + 2·Hkv, D]`` activation, RoPE rotates q and k in
place, and the varlen kernel reads q/k/v as strided views -- no concat, split,
``repeat_interleave`` or copy. Checkpoint keys stay ``q_proj/k_proj/v_proj``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable, Protocol

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.error import NotSupportedError
from fairseq2_b200.gang import Gangs
from fairseq2_b200.models.transformer.attention_bias import AttentionBiasCache
from fairseq2_b200.models.transformer.sdpa import SDPA
from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalState, IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm
from fairseq2_b200.nn.position_encoder import PositionEncoder
from fairseq2_b200.nn.projection import ColumnShardedLinear, Linear, Projection, RowShardedLinear
from fairseq2_b200.ops.gemm import linear as _linear
from fairseq2_b200.ops.tensor_parallel import reduce_on_backward
from fairseq2_b200.typing import DataType, Device


class AttentionWeightHook(Protocol):
    def __call__(self, m: "MultiheadAttention", attn: Tensor, attn_weights: Tensor) -> None: ...


class MultiheadAttention(Module, ABC):
    def __init__(self, model_dim: int, num_heads: int) -> None:
        super().__init__()
        self.model_dim, self.num_heads = model_dim, num_heads
        self._attn_weight_hooks: dict[int, AttentionWeightHook] = {}

    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, keys: Tensor, keys_layout: BatchLayout, values: Tensor,
                bias_cache: AttentionBiasCache, *, state_bag: IncrementalStateBag | None = None) -> Tensor: ...

    def register_attn_weight_hook(self, hook: AttentionWeightHook):  # type: ignore[no-untyped-def]
        key = max(self._attn_weight_hooks, default=-1) + 1
        self._attn_weight_hooks[key] = hook
        hooks = self._attn_weight_hooks

        class _Handle:
            def remove(self) -> None:
                hooks.pop(key, None)

        return _Handle()


class AttentionState(IncrementalState):
    @abstractmethod
    def append(self, k: Tensor, v: Tensor) -> None: ...

    @abstractmethod
    def get(self) -> tuple[Tensor, Tensor]: ...


class FullAttentionState(AttentionState):
    """Growable KV cache ``(N, capacity, Hkv, D)``; capacity grows in steps of
    ``capacity_increment`` up to ``max_seq_len``."""

    def __init__(self, k: Tensor, v: Tensor, max_seq_len: int, capacity_increment: int | None) -> None:
        n, s, h, d = k.shape
        self.max_seq_len = max_seq_len
        self.inc = capacity_increment
        cap = max_seq_len if capacity_increment is None else min(self._round(s), max_seq_len)
        self.k = k.new_empty((n, cap, h, d))
        self.v = v.new_empty((n, cap, h, d))
        self.k[:, :s], self.v[:, :s] = k, v
        self.seq_len = s

    def _round(self, n: int) -> int:
        assert self.inc is not None
        return ((n + self.inc - 1) // self.inc) * self.inc

    def append(self, k: Tensor, v: Tensor) -> None:
        s = k.shape[1]
        need = self.seq_len + s
        if need > self.k.shape[1]:
            if need > self.max_seq_len:
                raise ValueError(f"The KV cache cannot grow beyond the maximum sequence length ({self.max_seq_len}).")
            cap = min(self._round(need), self.max_seq_len) if self.inc is not None else self.max_seq_len
            nk = self.k.new_empty((self.k.shape[0], cap, *self.k.shape[2:]))
            nv = self.v.new_empty((self.v.shape[0], cap, *self.v.shape[2:]))
            nk[:, : self.seq_len], nv[:, : self.seq_len] = self.k[:, : self.seq_len], self.v[:, : self.seq_len]
            self.k, self.v = nk, nv
        self.k[:, self.seq_len:need], self.v[:, self.seq_len:need] = k, v
        self.seq_len = need

    def get(self) -> tuple[Tensor, Tensor]:
        return self.k[:, : self.seq_len], self.v[:, : self.seq_len]

    def reorder(self, new_order: Tensor) -> None:
        self.k = self.k.index_select(0, new_order)
        self.v = self.v.index_select(0, new_order)

    def size_bytes(self) -> int:
        return 2 * self.seq_len * self.k.shape[0] * self.k.shape[2] * self.k.shape[3] * self.k.element_size()

    def capacity_bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class LocalAttentionState(AttentionState):
    """Sliding-window KV cache holding the last ``attn_window_len`` positions."""

    def __init__(self, k: Tensor, v: Tensor, max_seq_len: int, attn_window_len: int,
                 capacity_increment: int | None) -> None:
        self.window = attn_window_len
        self.k = k[:, -attn_window_len:].clone()
        self.v = v[:, -attn_window_len:].clone()

    def append(self, k: Tensor, v: Tensor) -> None:
        self.k = torch.cat([self.k, k], dim=1)[:, -self.window:]
        self.v = torch.cat([self.v, v], dim=1)[:, -self.window:]

    def get(self) -> tuple[Tensor, Tensor]:
        return self.k, self.v

    def reorder(self, new_order: Tensor) -> None:
        self.k = self.k.index_select(0, new_order)
        self.v = self.v.index_select(0, new_order)

    def size_bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def capacity_bytes(self) -> int:
        return self.size_bytes()


class StaticAttentionState(AttentionState):
    """Encoder-decoder attention: keys/values are computed once."""

    def __init__(self, k: Tensor, v: Tensor, max_seq_len: int = 0, capacity_increment: int | None = None) -> None:
        self.k, self.v = k, v

    def append(self, k: Tensor, v: Tensor) -> None:
        raise ValueError("`StaticAttentionState` does not support `append()`.")

    def get(self) -> tuple[Tensor, Tensor]:
        return self.k, self.v

    def reorder(self, new_order: Tensor) -> None:
        if new_order.shape[0] != self.k.shape[0]:
            self.k = self.k.index_select(0, new_order)
            self.v = self.v.index_select(0, new_order)
        else:
            self.k = self.k.index_select(0, new_order)
            self.v = self.v.index_select(0, new_order)

    def size_bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def capacity_bytes(self) -> int:
        return self.size_bytes()


def _adjacent(ws: list[Tensor]) -> Tensor | None:
    """If the 2-D weights lie back to back in one storage return the merged view."""
    w0 = ws[0]
    if any(w.dtype != w0.dtype or w.device != w0.device or not w.is_contiguous() or w.shape[1] != w0.shape[1]
           for w in ws):
        return None
    try:
        st = w0.untyped_storage().data_ptr()
        if any(w.untyped_storage().data_ptr() != st for w in ws):
            return None
    except RuntimeError:
        return None
    off = w0.storage_offset()
    rows = 0
    for w in ws:
        if w.storage_offset() != off + rows * w0.shape[1]:
            return None
        rows += w.shape[0]
    return w0.as_strided((rows, w0.shape[1]), (w0.shape[1], 1), off)


class _MergedLinearFn(torch.autograd.Function):
    """One GEMM for several projections that share the input; weight grads are
    produced by one wgrad GEMM and handed out as views."""

    @staticmethod
    def forward(ctx, x: Tensor, merged: Tensor, *ws: Tensor) -> Tensor:  # type: ignore[override]
        from fairseq2_b200.ops.gemm import gemm

        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, merged)
        ctx.rows = [w.shape[0] for w in ws]
        ctx.x_shape = x.shape
        ctx.sinks = [getattr(w, "grad_sink", None) for w in ws]
        ctx.ws = ws
        return gemm(x2, merged).view(*x.shape[:-1], merged.shape[0])

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        from fairseq2_b200.ops.gemm import gemm

        x2, merged = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = gemm(dy2, merged, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        sink = _merged_sink(ctx.ws)
        if sink is not None:
            gemm(dy2, x2, a_mn=True, b_mn=True, out=sink[0], accumulate=sink[1])
            for w in ctx.ws:
                w.grad_sink_filled = True
            return (dx, None, *([None] * len(ctx.rows)))
        dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        return (dx, None, *dw.split(ctx.rows, dim=0))


def _merged_sink(ws) -> tuple[Tensor, bool] | None:  # type: ignore[no-untyped-def]
    sinks = [getattr(w, "grad_sink", None) for w in ws]
    if any(s is None for s in sinks):
        return None
    m = _adjacent(sinks)
    if m is None:
        return None
    filled = [bool(getattr(w, "grad_sink_filled", False)) for w in ws]
    if any(filled) and not all(filled):
        return None
    return m, all(filled)


def merged_linear(x: Tensor, projs: list[Projection]) -> Tensor | None:
    """Runs ``projs`` (plain or column-sharded linears without bias that share
    ``x``) as one GEMM when their weights are adjacent in memory; returns
    ``None`` when that is not possible."""
    ws = []
    sp_gang = None
    for p in projs:
        if not isinstance(p, (Linear, ColumnShardedLinear)) or p.bias is not None:
            return None
        if isinstance(p, ColumnShardedLinear) and p.gang.size > 1:
            # tensor parallel: only the sequence-parallel form merges (one all-gather of the token shard inside
            # ONE GEMM over the adjacent local weight shards instead of one collective per projection)
            if not p.sequence_parallel or p.gather_output or (sp_gang is not None and p.gang is not sp_gang):
                return None
            sp_gang = p.gang
        elif sp_gang is not None:
            return None
        ws.append(p.weight)
    if not x.is_cuda or x.dtype != torch.bfloat16:
        return None
    merged = _adjacent([w.detach() for w in ws])
    if merged is None:
        return None
    if sp_gang is not None:
        from fairseq2_b200.nn.projection import _fused_ops

        if any(isinstance(p, Linear) for p in projs):
            return None
        ops = _fused_ops(sp_gang, x, x.shape[0] if x.ndim == 2 else 0, x.shape[-1], merged)
        if ops is None:
            return None
        return ops.column(x, merged, tuple(ws))
    return _MergedLinearFn.apply(x, merged, *ws)


class StandardMultiheadAttention(MultiheadAttention):
    def __init__(self, model_dim: int, num_heads: int, sdpa: SDPA, *, head_dim: int | None = None,
                 num_key_value_heads: int | None = None, kv_dim: int | None = None,
                 q_proj: Projection | None = None, k_proj: Projection | None = None,
                 v_proj: Projection | None = None, qkv_proj_init_fn: Callable[[Linear], None] | None = None,
                 q_norm: LayerNorm | None = None, k_norm: LayerNorm | None = None,
                 pos_encoder: PositionEncoder | None = None, output_proj: Projection | None = None,
                 output_proj_init_fn: Callable[[Linear], None] | None = None, bias: bool = True,
                 output_proj_bias: bool | None = None, state_factory: Callable[..., AttentionState] | None = None,
                 qk_norm_over_heads: bool = False, gangs: Gangs | None = None, device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(model_dim, num_heads)
        nkv = num_key_value_heads if num_key_value_heads is not None else num_heads
        if num_heads % nkv:
            raise ValueError(f"`num_heads` ({num_heads}) must be a multiple of `num_key_value_heads` ({nkv}).")
        hd = head_dim if head_dim is not None else model_dim // num_heads
        kv_dim = kv_dim if kv_dim is not None else model_dim
        self.num_key_value_heads, self.head_dim, self.kv_dim = nkv, hd, kv_dim
        tp = gangs.tp if gangs is not None and gangs.tp.size > 1 else None
        self.tp_size = tp.size if tp is not None else 1
        self._tp_gang = tp
        if tp is not None and (num_heads % tp.size or nkv % tp.size):
            raise ValueError("`num_heads` and `num_key_value_heads` must be multiples of the tensor parallel size.")

        from fairseq2_b200.parallel.tp import sequence_parallel_enabled

        sp = tp is not None and sequence_parallel_enabled()
        self.sequence_parallel = sp

        def col(i: int, o: int) -> Projection:
            if tp is not None:
                return ColumnShardedLinear(tp, i, o, bias, gather_output=False, sequence_parallel=sp,
                                           init_fn=qkv_proj_init_fn, device=device, dtype=dtype)
            return Linear(i, o, bias, init_fn=qkv_proj_init_fn, device=device, dtype=dtype)

        self.q_proj = q_proj if q_proj is not None else col(model_dim, num_heads * hd)
        self.k_proj = k_proj if k_proj is not None else col(kv_dim, nkv * hd)
        self.v_proj = v_proj if v_proj is not None else col(kv_dim, nkv * hd)
        # OLMo-2 style: q/k norms span the whole projection (all heads) rather than one head
        self.qk_norm_over_heads = qk_norm_over_heads
        self._norm_full_dims: tuple[int, int] | None = None
        if qk_norm_over_heads and tp is not None:
            # The normalised vector is split over the ranks together with the heads: every rank keeps its slice of
            # the weight, and the mean of squares is taken over all slices (summed over the gang, see
            # `_norm_over_heads`). Only a norm without mean subtraction and bias can be split this way.
            from fairseq2_b200.nn.normalization import RMSNorm

            for norm in (q_norm, k_norm):
                if norm is not None and (not isinstance(norm, RMSNorm) or norm.bias is not None):
                    raise NotSupportedError(
                        "`qk_norm_over_heads` with tensor parallelism needs RMS norms without bias.")
            self._norm_full_dims = (num_heads * hd, nkv * hd)

            def split(norm: LayerNorm | None, full: int) -> LayerNorm | None:
                if norm is None:
                    return None
                if norm.normalized_shape != (full,):
                    raise ValueError(f"The q/k norm must span the whole projection ({full}), but spans "
                                     f"{norm.normalized_shape}.")
                w = norm.weight
                return RMSNorm(full // tp.size, bias=False, eps=norm.eps, elementwise_affine=w is not None,
                               init_fn=norm.init_fn, device=w.device if w is not None else device,
                               dtype=w.dtype if w is not None else dtype)

            q_norm, k_norm = split(q_norm, num_heads * hd), split(k_norm, nkv * hd)
        self.q_norm, self.k_norm = q_norm, k_norm
        if pos_encoder is not None and pos_encoder.encoding_dim != hd:
            raise ValueError(f"`pos_encoder.encoding_dim` must equal the head dimension ({hd}).")
        self.pos_encoder = pos_encoder
        self.sdpa = sdpa
        ob = bias if output_proj_bias is None else output_proj_bias
        if output_proj is not None:
            self.output_proj = output_proj
        elif tp is not None:
            self.output_proj = RowShardedLinear(tp, num_heads * hd, model_dim, ob, scatter_input=False,
                                                sequence_parallel=sp, init_fn=output_proj_init_fn, device=device,
                                                dtype=dtype)
        else:
            self.output_proj = Linear(num_heads * hd, model_dim, ob, init_fn=output_proj_init_fn, device=device,
                                      dtype=dtype)
        self.state_factory = state_factory

    @property
    def gang(self):  # type: ignore[no-untyped-def]
        """The tensor-parallel gang (``None`` without tensor parallelism)."""
        return self._tp_gang

    def get_shard_dims(self) -> list[tuple[Parameter, int]]:
        """Parameters of this module itself (not of its projections) that are split over the tensor-parallel gang:
        the weights of q/k norms that span all heads."""
        if self._norm_full_dims is None:
            return []
        return [(n.weight, 0) for n in (self.q_norm, self.k_norm) if n is not None and n.weight is not None]

    def _norm_over_heads(self, norm: LayerNorm, x: Tensor, full_dim: int) -> Tensor:
        """RMS norm over a vector of ``full_dim`` entries of which this rank holds a slice."""
        if self._norm_full_dims is None:
            return norm(x)
        from fairseq2_b200.ops.tensor_parallel import reduce_both_ways

        xf = x.float()
        sq = reduce_both_ways(xf.pow(2).sum(dim=-1, keepdim=True), self._tp_gang)
        y = (xf * torch.rsqrt(sq / full_dim + norm.eps)).type_as(x)
        return y * norm.weight if norm.weight is not None else y

    def _head_norm(self, norm: LayerNorm, x: Tensor) -> Tensor:
        """A per-head q/k norm has ONE weight vector for all heads. With the heads split over tensor-parallel ranks
        and replicated activations, a rank's gradient of that weight only covers its own heads, and nothing
        downstream sums replicated parameters over the gang: the weight therefore enters through an identity whose
        backward pass does. (With sequence-parallel activations every replicated parameter has a partial gradient
        and the data-parallel engine sums them all, this one included.)"""
        if self._tp_gang is None or self.sequence_parallel or norm.weight is None or not torch.is_grad_enabled():
            return norm(x)
        weight = reduce_on_backward(norm.weight, self._tp_gang)
        bias = reduce_on_backward(norm.bias, self._tp_gang) if norm.bias is not None else None
        return norm.apply_with(x, weight, bias)

    # ------------------------------------------------------------------ forward
    def forward(self, seqs, seqs_layout, keys, keys_layout, values, bias_cache, *, state_bag=None):  # type: ignore[override]
        H = self.num_heads // self.tp_size
        Hkv = self.num_key_value_heads // self.tp_size
        D = self.head_dim
        self_attn = keys is seqs and values is seqs
        q = k = v = None
        if self_attn and self.q_norm is None and self.k_norm is None:
            qkv = merged_linear(seqs, [self.q_proj, self.k_proj, self.v_proj])
            if qkv is not None:
                qkv = qkv.unflatten(-1, (H + 2 * Hkv, D))
                fused = self._fused_self_attention(qkv, seqs_layout, state_bag, H, Hkv)
                if fused is not None:
                    return self.output_proj(fused)
                q, k, v = qkv[..., :H, :], qkv[..., H:H + Hkv, :], qkv[..., H + Hkv:, :]
        if q is None:
            q = self.q_proj(seqs)
            if self.q_norm is not None and self.qk_norm_over_heads:
                q = self._norm_over_heads(self.q_norm, q, self.num_heads * self.head_dim)
            q = q.unflatten(-1, (H, D))
            if self.q_norm is not None and not self.qk_norm_over_heads:
                q = self._head_norm(self.q_norm, q)
        if self.pos_encoder is not None:
            q = self.pos_encoder(q, seqs_layout, state_bag=state_bag)

        static = isinstance(state_bag.maybe_get_state(self, AttentionState), StaticAttentionState) \
            if (state_bag is not None and not self.training) else False
        if static:
            k, v = state_bag.maybe_get_state(self, AttentionState).get()  # type: ignore[union-attr]
        else:
            if k is None:
                k = self.k_proj(keys)
                if self.k_norm is not None and self.qk_norm_over_heads:
                    k = self._norm_over_heads(self.k_norm, k, self.num_key_value_heads * self.head_dim)
                k = k.unflatten(-1, (Hkv, D))
                v = self.v_proj(values).unflatten(-1, (Hkv, D))
                if self.k_norm is not None and not self.qk_norm_over_heads:
                    k = self._head_norm(self.k_norm, k)
            if self.pos_encoder is not None:
                k = self.pos_encoder(k, keys_layout, state_bag=state_bag)
            if state_bag is not None and not self.training:
                state = state_bag.maybe_get_state(self, AttentionState)
                if state is None:
                    factory = self.state_factory or FullAttentionState
                    if not self_attn:
                        factory = StaticAttentionState
                    state = factory(k, v, state_bag.max_num_steps, state_bag.capacity_increment)
                    state_bag.set_state(self, state)
                else:
                    state.append(k, v)
                    k, v = state.get()
                    keys_layout = BatchLayout.of(k)
        needs_w = bool(self._attn_weight_hooks)
        attn, w = self.sdpa(q, seqs_layout, k, keys_layout, v, bias_cache, needs_weights=needs_w)
        if w is not None:
            for hook in self._attn_weight_hooks.values():
                hook(self, attn, w)
        return self.output_proj(attn.flatten(-2, -1))

    def _fused_self_attention(self, qkv: Tensor, layout: BatchLayout, state_bag: IncrementalStateBag | None,
                              H: int, Hkv: int) -> Tensor | None:
        """RoPE + attention straight on the merged projection output (training
        and cache-less inference on packed or padded batches)."""
        from fairseq2_b200.models.transformer.attention_bias import CausalAttentionBias, IdentityBias
        from fairseq2_b200.models.transformer.sdpa import VarlenSDPA
        from fairseq2_b200.nn.position_encoder import RotaryEncoder
        from fairseq2_b200.ops.attention import qkv_rope_attention

        if state_bag is not None or self._attn_weight_hooks or not isinstance(self.sdpa, VarlenSDPA):
            return None
        bias = self.sdpa.bias
        if not isinstance(bias, (CausalAttentionBias, IdentityBias)):
            return None
        window = getattr(bias, "attn_window_len", None)
        if window and self.head_dim != 128:        # the sliding window lives in the tcgen05 kernels only
            return None
        drop = self.sdpa.dropout_p if self.training else 0.0
        if drop > 0.0 and window:                  # dropout lives in the mma.sync kernels, the window in the others
            return None
        pe = self.pos_encoder
        if pe is not None and type(pe) is not RotaryEncoder:
            return None
        if self.head_dim not in (64, 128) or not qkv.is_contiguous():
            return None
        flat = qkv if layout.packed else qkv.flatten(0, 1)
        freqs = pos = None
        if pe is not None:
            if layout.max_seq_len > pe.max_seq_len:
                raise ValueError(
                    f"The lengths of all sequences in `seqs` must be less than or equal to the maximum sequence length ({pe.max_seq_len}).")
            freqs, pos = pe.freqs, layout.position_indices_i32.reshape(-1)
        out = qkv_rope_attention(flat, freqs, pos, layout.seq_begin_indices_pt[:-1], layout.seq_lens_pt,
                                 layout.max_seq_len, num_heads=H, num_kv_heads=Hkv,
                                 causal=isinstance(bias, CausalAttentionBias),
                                 has_padding=layout.padded or sum(layout.seq_lens) < flat.shape[0], window=window,
                                 dropout_p=drop)
        out = out.flatten(-2, -1)
        if not layout.packed:
            out = out.view(*qkv.shape[:2], H * self.head_dim)
        return out

    def extra_repr(self) -> str:
        return (f"model_dim={self.model_dim}, num_heads={self.num_heads}, "
                f"num_key_value_heads={self.num_key_value_heads}, head_dim={self.head_dim}")
