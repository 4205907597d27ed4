"""Fused pieces of the wav2vec 2.0 objective: contrastive loss over index-given distractors and the Gumbel
vector quantizer (fairseq2 ``models/wav2vec2/model.py:289-443``, ``vector_quantizer.py:80-200``).

Both avoid the large intermediates of the tensor formulation -- the gathered ``[N, S, K, M]`` distractor tensor and the
``[frames, G*V, E]`` product of one-hot codes with the code book -- and fall back to that formulation on CPU.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from fairseq2_b200.ops._ext import require_ext, use_kernels


# ------------------------------------------------------------------------------------------- contrastive loss
def contrastive_reference(x: Tensor, targets: Tensor, distractors: Tensor, temp: float) -> tuple[Tensor, Tensor]:
    """``x``, ``targets`` ``[P, M]``, ``distractors`` ``[P, K]`` rows of ``targets`` -> (logits [P, K+1] fp32, loss sum)."""
    cand = torch.cat([targets.unsqueeze(1), targets[distractors.long()]], dim=1)          # [P, K+1, M]
    logits = torch.cosine_similarity(x.float().unsqueeze(1), cand.float(), dim=-1) / temp
    same = (cand[:, 1:] == targets.unsqueeze(1)).all(-1)
    logits = torch.cat([logits[:, :1], logits[:, 1:].masked_fill(same, float("-inf"))], dim=1)
    loss = F.cross_entropy(logits, logits.new_zeros(logits.shape[0], dtype=torch.int64), reduction="sum")
    return logits, loss


class _ContrastiveFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, targets: Tensor, distractors: Tensor, temp: float):  # type: ignore[override]
        ext = require_ext()
        logits, lse, loss = ext.w2v_contrastive_fwd(x, targets, distractors, temp)
        ctx.save_for_backward(x, targets, distractors, logits, lse)
        ctx.temp = temp
        ctx.mark_non_differentiable(logits)
        return logits, loss.squeeze(0)

    @staticmethod
    def backward(ctx, _dlogits: Tensor, dloss: Tensor):  # type: ignore[override]
        ext = require_ext()
        x, targets, distractors, logits, lse = ctx.saved_tensors
        scale = dloss.detach().float().reshape(1).contiguous()
        dx, dt = ext.w2v_contrastive_bwd(x, targets, distractors, logits, lse, scale, ctx.temp)
        return dx.to(x.dtype), dt.to(targets.dtype), None, None


def contrastive_logits_and_loss(x: Tensor, targets: Tensor, distractors: Tensor, temp: float) -> tuple[Tensor, Tensor]:
    """Cosine-similarity logits against the true target (column 0) and ``K`` distractors, and the summed cross entropy.
    The logits are returned for metrics only (no gradient flows through them)."""
    if (use_kernels(x, targets) and x.dtype in (torch.bfloat16, torch.float32) and x.dtype == targets.dtype
            and x.shape[-1] <= 1024):
        return _ContrastiveFn.apply(x.contiguous(), targets.contiguous(), distractors.to(torch.int32).contiguous(), temp)
    return contrastive_reference(x, targets, distractors, temp)


# ------------------------------------------------------------------------------------------ Gumbel quantizer
def gumbel_quantize_reference(logits: Tensor, noise: Tensor | None, entries: Tensor, G: int, tau: float,
                              training: bool) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """``logits`` [R, V] (rows ordered (frame, codebook)), ``entries`` [G*V, E] -> (q [R, E], sel [R], prob_sum [G, V],
    hard_count [G, V]) with the straight-through gradient."""
    R, V = logits.shape
    lf = logits.float()
    hard_idx = lf.argmax(dim=-1)
    prob_sum = torch.softmax(lf, dim=-1).view(-1, G, V).sum(dim=0)
    hard_count = F.one_hot(hard_idx, V).float().view(-1, G, V).sum(dim=0)
    if training:
        z = (lf + (noise if noise is not None else 0.0)) / tau
        y = torch.softmax(z, dim=-1)
        sel = y.argmax(dim=-1)
        coeff = F.one_hot(sel, V).float() - y.detach() + y
    else:
        sel = hard_idx
        coeff = F.one_hot(sel, V).float()
    ent = entries.float().view(G, V, -1)
    q = torch.einsum("fgv,gve->fge", coeff.view(-1, G, V), ent).reshape(R, -1)
    return q.to(logits.dtype), sel, prob_sum, hard_count


class _GumbelQuantizeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: Tensor, noise: Tensor | None, entries: Tensor, G: int, tau: float, training: bool):  # type: ignore[override]
        ext = require_ext()
        q, hard_idx, sel, prob_sum, hard_count, y_soft = ext.w2v_quantize_fwd(logits, noise, entries, G, tau, training,
                                                                              True)
        ctx.save_for_backward(entries, y_soft, sel)
        ctx.G, ctx.tau, ctx.training, ctx.dtype = G, tau, training, logits.dtype
        ctx.mark_non_differentiable(sel, hard_count)
        return q, sel, prob_sum, hard_count

    @staticmethod
    def backward(ctx, dq: Tensor, _dsel: Tensor, _dprob: Tensor, _dhard: Tensor):  # type: ignore[override]
        if not ctx.training:
            return None, None, None, None, None, None
        ext = require_ext()
        entries, y_soft, sel = ctx.saved_tensors
        dlogits, dentries = ext.w2v_quantize_bwd(dq.contiguous(), entries, y_soft, sel, ctx.G, ctx.tau)
        return dlogits.to(ctx.dtype), None, dentries.to(entries.dtype), None, None, None


def gumbel_quantize(logits: Tensor, noise: Tensor | None, entries: Tensor, G: int, tau: float, training: bool
                    ) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """See ``gumbel_quantize_reference``. The soft-probability statistic ``prob_sum`` is differentiable through a
    PyTorch re-evaluation (it feeds the diversity loss); everything else comes from one kernel."""
    if (use_kernels(logits, entries) and logits.dtype in (torch.bfloat16, torch.float32)
            and logits.dtype == entries.dtype and logits.shape[-1] <= 512):
        q, sel, _, hard_count = _GumbelQuantizeFn.apply(logits.contiguous(), noise, entries.contiguous(), G, tau, training)
        prob_sum = torch.softmax(logits.float(), dim=-1).view(-1, G, logits.shape[-1]).sum(dim=0)
        return q, sel, prob_sum, hard_count
    return gumbel_quantize_reference(logits, noise, entries, G, tau, training)


def sample_gumbel_noise(shape: tuple[int, ...], device: torch.device, generator: torch.Generator | None = None) -> Tensor:
    u = torch.rand(shape, device=device, generator=generator).clamp_(1e-10, 1.0)
    return -torch.log((-torch.log(u)).clamp_(min=1e-10))
