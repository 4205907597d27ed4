"""Output projection fused with masked cross-entropy -- worklist row W8.

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
