"""Mixture-of-experts feed-forward network (cf. fairseq2 ``models/transformer/experts.py:85-369``,
``models/llama4/moe.py:24-157``).

The reference feeds EVERY token to EVERY expert with the non-selected ones
multiplied by ``sigmoid(-inf) = 0``, i.e. ``num_experts`` times the needed
FLOPs. Here tokens are dispatched sparsely: rows are permuted so that each
expert's tokens are contiguous, every expert runs one GEMM over exactly its
rows, and the results are combined with an index-add. Because the experts are
bias-free GLU networks, ``expert(0) = 0`` and the two formulations agree.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Any

import torch
from torch import Tensor
from torch.nn import Module, Parameter, SiLU

from fairseq2_b200.gang import Gang
from fairseq2_b200.models.transformer.ffn import FeedForwardNetwork, GLUFeedForwardNetwork
from fairseq2_b200.ops.grouped_gemm import grouped_mm, grouped_mm_device, grouped_mm_device_supported
from fairseq2_b200.ops.tensor_parallel import reduce, reduce_on_backward
from fairseq2_b200.typing import DataType, Device


class ExpertNetwork(Module, ABC):
    def __init__(self, num_experts: int, model_dim: int, inner_dim: int) -> None:
        super().__init__()
        self.num_experts, self.model_dim, self.inner_dim = num_experts, model_dim, inner_dim

    @abstractmethod
    def forward(self, x: Tensor, group_sizes: list[int]) -> Tensor:
        """``x``: ``[R, model_dim]`` rows sorted by expert, ``group_sizes[e]`` rows for expert ``e``."""

    @property
    def num_local_experts(self) -> int:
        return self.num_experts


class GroupedExpertNetwork(ExpertNetwork):
    """All experts' GLU weights stacked: ``gate_proj``/``inner_proj`` ``[E, D, F]``, ``output_proj`` ``[E, F, D]``."""

    def __init__(self, num_experts: int, model_dim: int, inner_dim: int, *, activation: Module | None = None,
                 device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(num_experts, model_dim, inner_dim)
        kw = {"device": device, "dtype": dtype}
        self.gate_proj = Parameter(torch.empty((num_experts, model_dim, inner_dim), **kw))
        self.inner_proj = Parameter(torch.empty((num_experts, model_dim, inner_dim), **kw))
        self.output_proj = Parameter(torch.empty((num_experts, inner_dim, model_dim), **kw))
        self.activation = activation if activation is not None else SiLU()
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for w in (self.gate_proj, self.inner_proj, self.output_proj):
            if w.device.type != "meta":
                torch.nn.init.trunc_normal_(w, std=w.shape[1] ** -0.5, a=-3 * w.shape[1] ** -0.5, b=3 * w.shape[1] ** -0.5)

    def forward(self, x: Tensor, group_sizes: list[int]) -> Tensor:
        h = self.activation(grouped_mm(x, self.gate_proj, group_sizes)) * grouped_mm(x, self.inner_proj, group_sizes)
        return grouped_mm(h, self.output_proj, group_sizes)

    def supports_padded_layout(self, x: Tensor) -> bool:
        return all(grouped_mm_device_supported(x, w) for w in (self.gate_proj, self.inner_proj, self.output_proj))

    def forward_padded(self, x: Tensor, layout: tuple[Tensor, Tensor, Tensor, Tensor]) -> Tensor:
        """``x`` in the 128-row padded expert-sorted layout: three single-launch grouped GEMMs, no host-side sizes."""
        g, u = grouped_mm_device(x, self.gate_proj, layout), grouped_mm_device(x, self.inner_proj, layout)
        if isinstance(self.activation, SiLU):
            from fairseq2_b200.ops.moe import swiglu_gate_up

            h = swiglu_gate_up(g, u, layout[3])                  # one pass over the rows that hold data
        else:
            h = self.activation(g) * u
        return grouped_mm_device(h, self.output_proj, layout)


class TPShardedExpertNetwork(ExpertNetwork):
    """Every expert's inner dimension is split over the tensor-parallel gang; the caller reduces the output."""

    def __init__(self, gang: Gang, num_experts: int, model_dim: int, inner_dim: int, *,
                 activation: Module | None = None, device: Device | None = None, dtype: DataType | None = None) -> None:
        super().__init__(num_experts, model_dim, inner_dim)
        if inner_dim % gang.size:
            raise ValueError(f"`inner_dim` ({inner_dim}) must be a multiple of the gang size ({gang.size}).")
        self.gang = gang
        f = inner_dim // gang.size
        kw = {"device": device, "dtype": dtype}
        self.gate_proj = Parameter(torch.empty((num_experts, model_dim, f), **kw))
        self.inner_proj = Parameter(torch.empty((num_experts, model_dim, f), **kw))
        self.output_proj = Parameter(torch.empty((num_experts, f, model_dim), **kw))
        self.activation = activation if activation is not None else SiLU()
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """This rank's slice of the unsplit initialisation, so that a tensor-parallel model equals its one-rank
        counterpart built from the same seed (as the sharded projections do)."""
        if self.gate_proj.device.type == "meta":
            return
        full = GroupedExpertNetwork(self.num_experts, self.model_dim, self.inner_dim, device=self.gate_proj.device,
                                    dtype=self.gate_proj.dtype)
        f, r = self.inner_dim // self.gang.size, self.gang.rank
        with torch.no_grad():
            self.gate_proj.copy_(full.gate_proj[:, :, r * f:(r + 1) * f])
            self.inner_proj.copy_(full.inner_proj[:, :, r * f:(r + 1) * f])
            self.output_proj.copy_(full.output_proj[:, r * f:(r + 1) * f, :])

    def get_shard_dims(self) -> list[tuple[Parameter, int]]:
        """(parameter, dimension split over the gang): what checkpoint resharding and the data-parallel engine go by."""
        return [(self.gate_proj, 2), (self.inner_proj, 2), (self.output_proj, 1)]

    @staticmethod
    def from_grouped_expert_network(net: GroupedExpertNetwork, gang: Gang) -> "TPShardedExpertNetwork":
        out = TPShardedExpertNetwork(gang, net.num_experts, net.model_dim, net.inner_dim, activation=net.activation,
                                     device=net.gate_proj.device, dtype=net.gate_proj.dtype)
        f, r = net.inner_dim // gang.size, gang.rank
        with torch.no_grad():
            out.gate_proj.copy_(net.gate_proj[:, :, r * f:(r + 1) * f])
            out.inner_proj.copy_(net.inner_proj[:, :, r * f:(r + 1) * f])
            out.output_proj.copy_(net.output_proj[:, r * f:(r + 1) * f, :])
        return out

    def forward(self, x: Tensor, group_sizes: list[int]) -> Tensor:
        h = self.activation(grouped_mm(x, self.gate_proj, group_sizes)) * grouped_mm(x, self.inner_proj, group_sizes)
        return grouped_mm(h, self.output_proj, group_sizes)


def route_tokens(logits: Tensor, top_k: int, softmax_gate: bool = False) -> tuple[Tensor, Tensor, Tensor, list[int]]:
    """Token-choice routing. Returns ``(token_idx [R], expert_scores [R], order, group_sizes)`` where the ``R = T·k``
    routed rows are sorted by expert; ``expert_scores`` is ``sigmoid`` of the selected logits, or their softmax
    over the ``top_k`` choices of the token with ``softmax_gate``."""
    T, E = logits.shape
    scores, experts = torch.topk(logits, top_k, dim=1)                   # [T, k]
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)                           # rows grouped by expert
    token_idx = order // top_k
    sizes = torch.bincount(flat_e, minlength=E).tolist()
    gates = torch.softmax(scores.float(), dim=1) if softmax_gate else torch.sigmoid(scores.float())
    return token_idx, gates.reshape(-1)[order], order, sizes


class MoE(FeedForwardNetwork):
    """Top-k routed experts plus an optional always-on shared expert (LLaMA-4)."""

    def __init__(self, model_dim: int, inner_dim: int, use_shared_expert: bool, num_experts: int,
                 capacity_factor: float, top_k: int, *, moe_activation: Module | None = None,
                 inner_dim_scale: float = 2 / 3, inner_dim_to_multiple: int = 1, auto_scale: bool = True,
                 tp_gang: Gang | None = None, ep: Any | None = None, softmax_gate: bool = False,
                 aux_loss: bool = False, router_init_std: float | None = None, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        """``ep``: an ``ops.moe_ep.ExpertParallelExchange``. When given, this rank holds only its
        ``num_experts / ep.arena.world`` experts and tokens travel to the owning rank inside the dispatch kernel and
        back inside the combine kernel; the router and the shared expert stay replicated.

        ``softmax_gate``: gates are the softmax over the selected ``top_k`` logits (Mixtral / Qwen-MoE style)
        instead of independent sigmoids (LLaMA 4). ``aux_loss``: every forward pass in training mode leaves the
        router's load-balancing loss in ``self.last_aux_loss`` (see ``ops.moe.load_balancing_loss``) for the model
        to add to its objective. ``router_init_std``: normal initialisation of the router (default
        ``model_dim ** -0.5``, truncated)."""
        super().__init__(model_dim)
        if inner_dim_scale != 1.0:
            inner_dim = int(inner_dim * inner_dim_scale)
        if auto_scale:
            # keep the activated parameter count equal to that of a dense layer
            inner_dim = int(inner_dim / (capacity_factor + int(use_shared_expert)))
        if inner_dim_to_multiple != 1:
            inner_dim = inner_dim_to_multiple * ((inner_dim + inner_dim_to_multiple - 1) // inner_dim_to_multiple)
        self.inner_dim, self.num_experts, self.top_k = inner_dim, num_experts, top_k
        self.tp_gang = tp_gang if tp_gang is not None and tp_gang.size > 1 else None
        self.shared_expert: GLUFeedForwardNetwork | None = None
        if use_shared_expert:
            shared_gangs = None
            if self.tp_gang is not None:
                # the shared expert is split over the inner dimension like any FFN (its output projection sums over
                # the gang itself)
                from fairseq2_b200.gang import FakeGang, Gangs

                one = FakeGang(self.tp_gang.device)
                shared_gangs = Gangs(root=self.tp_gang, dp=one, rdp=one, sdp=one, tp=self.tp_gang, pp=one)
            self.shared_expert = GLUFeedForwardNetwork(model_dim, inner_dim, bias=False, inner_dim_scale=1.0,
                                                       gangs=shared_gangs, device=device, dtype=dtype)
        self.router = Parameter(torch.empty((model_dim, num_experts), device=device, dtype=dtype))
        self.softmax_gate, self.aux_loss, self.router_init_std = softmax_gate, aux_loss, router_init_std
        self.last_aux_loss: Tensor | None = None
        self.ep = ep
        if ep is not None:
            if self.tp_gang is not None:
                raise ValueError("Expert parallelism and tensor-parallel experts are mutually exclusive.")
            if ep.num_experts != num_experts or ep.model_dim != model_dim:
                raise ValueError("`ep` was created for a different number of experts or model dimension.")
            self.experts: ExpertNetwork = GroupedExpertNetwork(ep.num_local_experts, model_dim, inner_dim,
                                                               activation=moe_activation, device=device, dtype=dtype)
        elif self.tp_gang is not None:
            self.experts = TPShardedExpertNetwork(self.tp_gang, num_experts, model_dim, inner_dim,
                                                  activation=moe_activation, device=device, dtype=dtype)
        else:
            self.experts = GroupedExpertNetwork(num_experts, model_dim, inner_dim, activation=moe_activation,
                                                device=device, dtype=dtype)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.router.device.type != "meta":
            if self.router_init_std is not None:
                torch.nn.init.normal_(self.router, std=self.router_init_std)
            else:
                torch.nn.init.trunc_normal_(self.router, std=self.model_dim ** -0.5)

    def _router_logits(self, x: Tensor) -> Tensor:
        """``x @ router`` on the tcgen05 GEMM (the router is stored ``[D, E]``, i.e. as an MN-major B operand)."""
        from fairseq2_b200.ops.gemm import linear_kn

        return linear_kn(x, self.router, out_dtype=torch.float32 if x.is_cuda else None)

    def _note_aux_loss(self, logits: Tensor, counts: Tensor) -> None:
        from fairseq2_b200.ops.moe import load_balancing_loss

        self.last_aux_loss = load_balancing_loss(logits, counts, self.top_k) \
            if (self.aux_loss and self.training) else None

    def forward(self, seqs: Tensor) -> Tensor:
        x = seqs.reshape(-1, self.model_dim)
        logits = self._router_logits(x)
        from fairseq2_b200.ops import moe as moe_ops

        if self.ep is not None:
            if not moe_ops.moe_kernels_available(x, logits):
                raise RuntimeError("Expert parallelism needs the CUDA routing kernels (bf16 activations on a GPU).")
            ids, gates, counts = moe_ops.moe_route(logits, self.top_k, self.softmax_gate)
            self._note_aux_loss(logits, counts)
            if isinstance(self.experts, GroupedExpertNetwork) and self.experts.supports_padded_layout(x):
                # tile-aligned inbox + device-resident tile tables: three single-launch grouped GEMMs, and the
                # host never waits for the routing result
                rows, dest, layout, _ = self.ep.dispatch_padded(x, ids, counts, gates=gates)
                rows_out = self.experts.forward_padded(rows, layout)
                num_tiles = layout[3]
            else:
                rows, dest, group_sizes = self.ep.dispatch(x, ids, counts, gates=gates)
                rows_out = self.experts(rows, group_sizes.tolist())
                num_tiles = None
            base = self.shared_expert(x) if self.shared_expert is not None else None
            return self.ep.combine(rows_out, dest, x.shape[0], base=base, num_tiles=num_tiles).view(seqs.shape)
        # Tensor-parallel experts: every rank holds a slice of each expert's inner dimension, so the routed output is
        # a partial sum (summed over the gang below) and so is the gradient that the experts send back into `x`
        # (summed over the gang in the backward pass of `xe`). The shared expert does both inside its own sharded
        # projections and is added after the sum, not before: its output is already whole on every rank.
        xe = reduce_on_backward(x, self.tp_gang) if self.tp_gang is not None else x
        if moe_ops.moe_kernels_available(x, logits):
            # fused top-k gate + histogram, gather/scale into expert order, experts, gather back per token
            ids, gates, counts = moe_ops.moe_route(logits, self.top_k, self.softmax_gate)
            self._note_aux_loss(logits, counts)
            if self.tp_gang is not None:
                gates = reduce_on_backward(gates, self.tp_gang)      # the gates scale the experts' inputs: same story
            if isinstance(self.experts, GroupedExpertNetwork) and self.experts.supports_padded_layout(x):
                # padded layout + device-resident tile tables: the CPU never waits for the routing result
                routed_in, src_row, inv, layout = moe_ops.moe_dispatch_padded(xe, gates, ids, counts)
                routed_out = self.experts.forward_padded(routed_in, layout)
            else:
                routed_in, src_row, inv = moe_ops.moe_dispatch(xe, gates, ids, counts)
                routed_out = self.experts(routed_in, counts.tolist())
            base = self.shared_expert(x) if self.shared_expert is not None else None
            if self.tp_gang is None:
                return moe_ops.moe_combine(routed_out, inv, src_row, base).view(seqs.shape)
            out = reduce(moe_ops.moe_combine(routed_out, inv, src_row, None), self.tp_gang)
            return (out if base is None else out + base).view(seqs.shape)
        token_idx, scores, _, sizes = route_tokens(logits, self.top_k, self.softmax_gate)
        self._note_aux_loss(logits, torch.tensor(sizes, device=logits.device))
        if self.tp_gang is not None:
            scores = reduce_on_backward(scores, self.tp_gang)        # the gates scale the experts' inputs: same story
        routed_in = xe.index_select(0, token_idx) * scores.to(x.dtype).unsqueeze(1)
        routed_out = self.experts(routed_in, sizes)
        out = torch.zeros_like(x).index_add(0, token_idx, routed_out)
        if self.tp_gang is not None:
            out = reduce(out, self.tp_gang)
        if self.shared_expert is not None:
            out = out + self.shared_expert(x)
        return out.view(seqs.shape)

    def extra_repr(self) -> str:
        return (f"model_dim={self.model_dim}, inner_dim={self.inner_dim}, num_experts={self.num_experts}, "
                f"top_k={self.top_k}")
