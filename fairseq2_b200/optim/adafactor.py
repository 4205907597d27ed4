"""Adafactor (Shazeer & Stern 2018) with the hyper-parameters and update rule of ``torch.optim.Adafactor``, which
is what the reference's ``optimizer.name = adafactor`` builds (fairseq2 ``recipe/config.py:851-897``,
``recipe/internal/optim.py``): factored second moments for matrices (one running row vector and one running
column vector instead of a full matrix), relative step size ``max(eps2, rms(p)) * min(lr, 1/sqrt(t))``, update
clipping by ``d``.

Besides plain parameters it understands the dim-0 shards of an FSDP unit (parameters that carry ``_fs2_unit``):
their gradient is a view of the unit's reduced gradient shard, the deferred gradient scale (loss normalisation x
clip factor) is applied on the fly, and every statistic that spans the rows of the full parameter -- column
means, the parameter RMS, the norm of the update -- is summed over the shard gang, so a sharded run follows the
unsharded one.
"""
from __future__ import annotations

from typing import Any, Callable, Iterable

import torch
from torch import Tensor
from torch.optim import Optimizer

from fairseq2_b200.gang import ReduceOperation


class Adafactor(Optimizer):
    def __init__(self, params: Iterable[Any], lr: float = 1e-2, beta2_decay: float = -0.8,
                 eps: tuple[float | None, float] = (None, 1e-3), d: float = 1.0, weight_decay: float = 0.0,
                 *, foreach: bool | None = None, maximize: bool = False) -> None:
        if lr < 0.0:
            raise ValueError(f"`lr` must be non-negative, but is {lr} instead.")
        if beta2_decay > 0.0:
            raise ValueError(f"`beta2_decay` must be non-positive, but is {beta2_decay} instead.")
        if d < 1.0:
            raise ValueError(f"`d` must be greater than or equal to 1, but is {d} instead.")
        eps = tuple(eps)  # type: ignore[assignment]
        super().__init__(params, dict(lr=lr, beta2_decay=beta2_decay, eps=eps, d=d, weight_decay=weight_decay,
                                      maximize=maximize))

    @staticmethod
    def _all_sum(t: Tensor, gang: Any) -> Tensor:
        if gang is not None and gang.size > 1:
            gang.all_reduce(t, ReduceOperation.SUM)
        return t

    @torch.no_grad()
    def step(self, closure: Callable[[], Tensor] | None = None, *, grad_scale: Tensor | None = None) -> Tensor | None:  # type: ignore[override]
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        touched_units: dict[int, Any] = {}
        for group in self.param_groups:
            lr, decay, (eps1, eps2), d = float(group["lr"]), group["beta2_decay"], group["eps"], group["d"]
            wd, maximize = group["weight_decay"], group["maximize"]
            for p in group["params"]:
                unit = getattr(p, "_fs2_unit", None)
                gang, full_rows = None, p.shape[0] if p.ndim > 0 else 1
                if unit is not None:
                    if not unit.grads_ready or unit.grad_shard is None:
                        continue
                    s = p._fs2_spec  # type: ignore[attr-defined]
                    took = getattr(unit, "took_part", None)
                    if took is not None and not took[unit.specs.index(s)]:
                        continue
                    n = s.rows_local * s.row
                    grad = unit.grad_shard[s.shard_off: s.shard_off + n].view(p.shape).to(p.device, torch.float32)
                    gang, full_rows = unit.gang, s.d0
                    touched_units[id(unit)] = unit
                elif p.grad is None:
                    continue
                else:
                    grad = p.grad.float()
                if grad_scale is not None:
                    grad = grad * grad_scale.to(grad.device)
                if maximize:
                    grad = -grad
                st = self.state[p]
                if not st:
                    st["step"] = torch.zeros((), dtype=torch.float32)
                    if p.ndim > 1:
                        st["row_var"] = torch.zeros(p.shape[:-1] + (1,), dtype=torch.float32, device=p.device)
                        st["col_var"] = torch.zeros(p.shape[:-2] + (1, p.shape[-1]), dtype=torch.float32,
                                                    device=p.device)
                    else:
                        st["variance"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                t = float(st["step"])
                e1 = torch.finfo(p.dtype).eps if eps1 is None else eps1
                beta2_t = 1.0 - t ** decay
                rho_t = min(lr, 1.0 / (t ** 0.5))
                # ---- relative step size from the RMS of the (full) parameter
                full_numel = s.d0 * s.row if unit is not None else p.numel()
                sq = self._all_sum(p.float().pow(2).sum(), gang)
                alpha = torch.clamp((sq / max(full_numel, 1)).sqrt(), min=eps2) * rho_t
                if wd != 0.0:
                    p.mul_(1.0 - lr * wd)
                g2 = grad * grad
                if p.ndim > 1:
                    row_var, col_var = st["row_var"], st["col_var"]
                    row_var.lerp_(g2.mean(dim=-1, keepdim=True), 1.0 - beta2_t)
                    # a column mean spans the rows of every shard (dim 0 is the sharded one only for matrices
                    # whose leading dimension is the row dimension; higher-rank parameters keep dim 0 as batch)
                    col_sum = g2.sum(dim=-2, keepdim=True)
                    rows = p.shape[-2]
                    if gang is not None and p.ndim == 2:
                        col_sum = self._all_sum(col_sum, gang)
                        rows = full_rows
                    col_var.lerp_(col_sum / max(rows, 1), 1.0 - beta2_t)
                    rv_sum = row_var.sum(dim=-2, keepdim=True)
                    if gang is not None and p.ndim == 2:
                        rv_sum = self._all_sum(rv_sum.clone(), gang)
                    rv_mean = (rv_sum / max(rows, 1)).clamp_(min=e1 * e1)
                    var_est = (row_var @ col_var) / rv_mean
                else:
                    st["variance"].lerp_(g2, 1.0 - beta2_t)
                    var_est = st["variance"].clone()
                update = var_est.clamp_(min=e1 * e1).rsqrt_().mul_(grad)
                usq = self._all_sum(update.pow(2).sum(), gang)
                denom = torch.clamp(usq.sqrt() / ((max(full_numel, 1) ** 0.5) * d), min=1.0)
                p.add_(update * (-alpha / denom).to(p.dtype))
        for unit in touched_units.values():
            unit.low_shard.copy_(unit.master, non_blocking=True)
        return loss
