"""Output projection fused with masked cross-entropy.

``fused_linear_cross_entropy`` never materialises the ``[T, V]`` logits of the
whole batch: tokens are processed in chunks; per chunk the tcgen05 GEMM writes
bf16 logits, one kernel turns them in place into ``(softmax - onehot) * mask``
while accumulating the fp32 loss on the device, and the dgrad/wgrad GEMMs
consume that buffer at once. The gradients w.r.t. the hidden states and the
projection weight are therefore produced in the forward pass and merely scaled
by the incoming gradient in backward.

Semantics follow fairseq2 ``nn/functional/cross_entropy.py:16-185``
(``log_softmax`` in fp32, ``pad_idx`` ignored, optional ``target_mask``,
reductions sum/mean).
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels
from fairseq2_b200.ops.gemm import gemm


def cross_entropy_reference(logits: Tensor, targets: Tensor, pad_idx: int | None = None, *,
                            target_mask: Tensor | None = None, label_smoothing: float = 0.0,
                            reduction: str = "sum") -> Tensor:
    lp = F.log_softmax(logits.float(), dim=-1)
    lp2 = lp.reshape(-1, lp.shape[-1])
    t = targets.reshape(-1)
    ignore = pad_idx if pad_idx is not None else -100
    nll = F.nll_loss(lp2, t, ignore_index=ignore, reduction="none")
    if label_smoothing > 0.0:
        # fairseq-compatible smoothing: (1 - ls - e) * nll + e * sum(-log p) with e = ls / (V - 1).
        smooth = -lp2.sum(dim=-1)
        if pad_idx is not None:
            smooth = smooth.masked_fill(t == pad_idx, 0.0)
        eps_i = label_smoothing / (lp2.shape[-1] - 1)
        nll = (1.0 - label_smoothing - eps_i) * nll + eps_i * smooth
    if target_mask is not None:
        nll = nll * target_mask.reshape(-1).to(nll.dtype)
    if reduction == "sum":
        return nll.sum()
    if reduction == "mean":
        if target_mask is not None:
            return nll.sum() / target_mask.sum().clamp(min=1)
        if pad_idx is not None:
            return nll.sum() / (t != pad_idx).sum().clamp(min=1)
        return nll.mean()
    if reduction == "none":
        return nll.view(targets.shape)
    raise ValueError(f"`reduction` must be 'sum', 'mean' or 'none', but is '{reduction}' instead.")


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h: Tensor, weight: Tensor, targets: Tensor, mask: Tensor | None, pad_idx: int,
                chunk: int) -> Tensor:  # type: ignore[override]
        ext = require_ext()
        T, D = h.shape
        V = weight.shape[0]
        loss = torch.zeros((), dtype=torch.float32, device=h.device)
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        dh = torch.empty_like(h) if need_dh else None
        dw = torch.zeros((V, D), dtype=torch.float32, device=h.device) if need_dw else None
        logits = torch.empty((min(chunk, T), V), dtype=torch.bfloat16, device=h.device)
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            lg = logits[: e - s]
            gemm(h[s:e], weight, out=lg)
            ext.ce_fwd_bwd_inplace(lg, targets[s:e], mask[s:e] if mask is not None else None, pad_idx, loss)
            if need_dh:
                gemm(lg, weight, b_mn=True, out=dh[s:e])
            if need_dw:
                gemm(lg, h[s:e], a_mn=True, b_mn=True, out=dw, accumulate=True)
        ctx.save_for_backward(dh, dw)
        ctx.wdtype = weight.dtype
        return loss

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        dh, dw = ctx.saved_tensors
        gdh = gdw = None
        if dh is not None:
            gdh = dh.mul_(g.to(dh.dtype))
        if dw is not None:
            gdw = (dw * g).to(ctx.wdtype)
        return gdh, gdw, None, None, None, None


def fused_linear_cross_entropy(h: Tensor, weight: Tensor, targets: Tensor, *, target_mask: Tensor | None = None,
                               pad_idx: int | None = None, reduction: str = "sum", chunk_size: int = 4096) -> Tensor:
    """Loss of ``cross_entropy(h @ weightᵀ, targets)`` without keeping the logits.

    ``h``: ``[..., D]``, ``weight``: ``[V, D]``, ``targets``: int64 ``[...]``,
    ``target_mask``: bool/float ``[...]``. Returns an fp32 scalar.
    """
    h2 = h.reshape(-1, h.shape[-1])
    t = targets.reshape(-1)
    m = target_mask.reshape(-1) if target_mask is not None else None
    if use_kernels(h2, weight) and h2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 \
            and weight.shape[0] % 8 == 0 and reduction in ("sum", "mean"):
        if m is not None and m.dtype != torch.float32:
            m = m.to(torch.float32)
        loss = _FusedLinearCE.apply(h2.contiguous(), weight, t.contiguous(), m, -100 if pad_idx is None else pad_idx,
                                    chunk_size)
        if reduction == "mean":
            if m is not None:
                denom = m.sum().clamp(min=1)
            elif pad_idx is not None:
                denom = (t != pad_idx).sum().clamp(min=1)
            else:
                denom = torch.tensor(float(t.numel()), device=h.device)
            loss = loss / denom
        return loss
    logits = F.linear(h2, weight)
    return cross_entropy_reference(logits, t, pad_idx, target_mask=m, reduction=reduction)


class _VocabParallelLinearCE(torch.autograd.Function):
    """Output projection + cross entropy with the vocabulary split over a tensor-parallel gang.

    Per chunk of rows every rank computes its ``[rows, V/W]`` slice of the logits and three per-row scalars -- the
    local maximum, the local sum of exponentials and the target logit if the target falls into its slice -- which
    are combined with one MAX and one SUM all-reduce of ``[rows]`` / ``[rows, 2]`` values. Neither the full logits
    nor the full vocabulary ever exist on one rank; gradients are produced in the same pass and scaled by the
    upstream gradient in backward (``dh`` is summed over the gang there, since every rank holds a partial)."""

    @staticmethod
    def forward(ctx, h: Tensor, weight: Tensor, targets: Tensor, mask: Tensor | None, pad_idx: int, chunk: int,
                gang: Any, reduce_dh: bool = True) -> Tensor:  # type: ignore[override]
        from fairseq2_b200.gang import ReduceOperation

        T, D = h.shape
        Vl = weight.shape[0]
        lo = gang.rank * Vl
        loss = torch.zeros((), dtype=torch.float32, device=h.device)
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh = torch.empty_like(h) if need_dh else None
        dw = torch.zeros((Vl, D), dtype=torch.float32, device=h.device) if need_dw else None
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            hc, tc = h[s:e], targets[s:e]
            logits = gemm(hc, weight, out_dtype=torch.float32) if hc.is_cuda else hc.float() @ weight.float().t()
            logits = logits.float()
            row_w = torch.ones(e - s, device=h.device) if mask is None else mask[s:e].float()
            if pad_idx >= 0:
                row_w = row_w * (tc != pad_idx)
            mx = logits.max(dim=1).values
            gang.all_reduce(mx, ReduceOperation.MAX)
            ex = torch.exp(logits - mx.unsqueeze(1))
            local = (tc >= lo) & (tc < lo + Vl)
            idx = (tc - lo).clamp(0, Vl - 1)
            stats = torch.stack([ex.sum(dim=1), torch.where(local, logits.gather(1, idx.unsqueeze(1)).squeeze(1),
                                                            torch.zeros_like(mx))], dim=1)
            gang.all_reduce(stats, ReduceOperation.SUM)
            loss += ((torch.log(stats[:, 0]) + mx - stats[:, 1]) * row_w).sum()
            if need_dh or need_dw:
                p = ex / stats[:, :1]
                p[torch.arange(e - s, device=h.device)[local], idx[local]] -= 1.0
                g = (p * row_w.unsqueeze(1)).to(h.dtype)
                if need_dh:
                    dh[s:e] = gemm(g, weight, b_mn=True) if g.is_cuda and g.dtype == torch.bfloat16 else \
                        (g.float() @ weight.float()).to(h.dtype)
                if need_dw:
                    dw += g.float().t() @ hc.float()
        ctx.save_for_backward(dh, dw)
        ctx.gang, ctx.wdtype, ctx.reduce_dh = gang, weight.dtype, reduce_dh
        return loss

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        from fairseq2_b200.gang import ReduceOperation

        dh, dw = ctx.saved_tensors
        gdh = gdw = None
        if dh is not None:
            gdh = dh.mul_(g.to(dh.dtype))
            if ctx.reduce_dh:
                ctx.gang.all_reduce(gdh, ReduceOperation.SUM)     # every rank contributed its vocabulary slice
        if dw is not None:
            gdw = (dw * g).to(ctx.wdtype)
        return gdh, gdw, None, None, None, None, None, None


def vocab_parallel_linear_cross_entropy(h: Tensor, weight_shard: Tensor, targets: Tensor, gang: Any, *,
                                        target_mask: Tensor | None = None, pad_idx: int | None = None,
                                        reduction: str = "sum", chunk_size: int = 4096,
                                        reduce_input_grad: bool = True) -> Tensor:
    """``cross_entropy(h @ concat_r(weight_shard_r)ᵀ, targets)`` where rank ``r`` of ``gang`` holds rows
    ``[r·V/W, (r+1)·V/W)`` of the output projection. Returns the same fp32 scalar on every rank.
    ``reduce_input_grad=False`` leaves the gradient of ``h`` as this rank's partial (its vocabulary slice's
    contribution) for a caller whose own backward sums over the gang, e.g. the reduce-scatter that is the backward
    of a sequence-parallel all-gather."""
    h2 = h.reshape(-1, h.shape[-1]).contiguous()
    t = targets.reshape(-1).contiguous()
    m = target_mask.reshape(-1).float() if target_mask is not None else None
    loss = _VocabParallelLinearCE.apply(h2, weight_shard, t, m, -100 if pad_idx is None else pad_idx, chunk_size,
                                        gang, reduce_input_grad)
    if reduction == "mean":
        denom = m.sum() if m is not None else ((t != pad_idx).sum() if pad_idx is not None
                                               else torch.tensor(float(t.numel()), device=h.device))
        loss = loss / denom.clamp(min=1)
    elif reduction != "sum":
        raise ValueError(f"`reduction` must be 'sum' or 'mean', but is '{reduction}' instead.")
    return loss
