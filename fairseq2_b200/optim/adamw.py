"""AdamW with a fused sm_100a step and first-class support for flat, sharded
parameter units.

Plain parameters are updated by the multi-tensor kernel of ``ops.optim`` (or
the PyTorch formulation on CPU). Parameters that are dim-0 shards of an FSDP
unit (they carry ``_fs2_unit``) are updated *per unit* with ONE launch over the
unit's flat fp32 master / moment buffers, reading the unit's reduced gradient
shard and refreshing its bf16 shard in the same pass: the optimizer half of
the fused reduce-scatter + update. ``grad_scale`` (loss normalisation x clip coefficient) is a
device scalar consumed inside the kernel.

Hyper-parameters and state layout (``step``, ``exp_avg``, ``exp_avg_sq`` per
parameter) follow ``torch.optim.AdamW`` so optimizer state dicts keep the
reference checkpoint format (fairseq2 ``recipe/internal/optim.py:61-72``).
"""
from __future__ import annotations

from typing import Any, Callable, Iterable

import torch
from torch import Tensor
from torch.optim import Optimizer

from fairseq2_b200.ops.optim import adamw_reference, multi_tensor_adamw


def _refresh_status_guard(param_groups: list[dict[str, Any]]) -> None:
    """The fused update kernels skip their work when a collective of this step gave up on a peer; they read a
    device-memory copy of the status word, which is brought up to date here, once per step."""
    for group in param_groups:
        for p in group["params"]:
            unit = getattr(p, "_fs2_unit", None)
            dev = unit.low_shard.device if unit is not None else p.device
            if dev.type == "cuda":
                from fairseq2_b200.ops._ext import require_ext, use_kernels

                if use_kernels(unit.low_shard if unit is not None else p):
                    require_ext().refresh_status_guard(dev.index if dev.index is not None else
                                                       torch.cuda.current_device())
            return


class AdamW(Optimizer):
    def __init__(self, params: Iterable[Any], lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, *, impl: str = "auto") -> None:
        if lr < 0.0:
            raise ValueError(f"`lr` must be non-negative, but is {lr} instead.")
        if not 0.0 <= betas[0] < 1.0 or not 0.0 <= betas[1] < 1.0:
            raise ValueError(f"`betas` must be in [0, 1), but are {betas} instead.")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.impl = impl
        self._unit_state: dict[int, tuple[Tensor, Tensor]] = {}

    def _unit_moments(self, unit: Any) -> tuple[Tensor, Tensor]:
        st = self._unit_state.get(id(unit))
        if st is None:
            st = (torch.zeros_like(unit.master), torch.zeros_like(unit.master))
            self._unit_state[id(unit)] = st
        return st

    def _init_state(self, p: Tensor) -> dict[str, Any]:
        st = self.state[p]
        if not st:
            unit = getattr(p, "_fs2_unit", None)
            st["step"] = torch.zeros((), dtype=torch.float32)
            if unit is not None:
                m, v = self._unit_moments(unit)
                s = p._fs2_spec  # type: ignore[attr-defined]
                n = s.rows_local * s.row
                st["exp_avg"] = m[s.shard_off: s.shard_off + n].view(p.shape)
                st["exp_avg_sq"] = v[s.shard_off: s.shard_off + n].view(p.shape)
            else:
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
        return st

    def prepare_fused_step(self, grad_scale: Tensor | None = None) -> int:
        """Arms the FSDP units of this optimizer so that their gradient reduce-scatter applies THIS step's update in
        the same kernel (``comm_reducescatter_adamw``): call before the backward pass, then :meth:`step` as usual
        afterwards -- it only has to book-keep for the units that were updated on the way. ``grad_scale`` is the
        device scalar (loss normalisation) multiplied into the averaged gradient. Returns the number of armed
        units. Only valid when no decision depends on all gradients at once (no clipping by the global norm, no
        loss-scale overflow check)."""
        armed = 0
        _refresh_status_guard(self.param_groups)
        for group in self.param_groups:
            b1, b2 = group["betas"]
            units: dict[int, Any] = {}
            for p in group["params"]:
                unit = getattr(p, "_fs2_unit", None)
                if unit is not None:
                    units[id(unit)] = unit
                    self._init_state(p)
            for unit in units.values():
                if unit.arena is None or unit.low_shard.dtype != torch.bfloat16 or unit.master.device != unit.device:
                    continue
                st0 = self.state[unit.shard_params[0]]
                step = st0.get("_host_step", int(st0["step"].item())) + 1
                m, v = self._unit_moments(unit)
                unit.fused_step = {"m": m, "v": v, "lr": float(group["lr"]), "beta1": b1, "beta2": b2,
                                   "eps": group["eps"], "weight_decay": group["weight_decay"], "step": step,
                                   "grad_scale": grad_scale}
                unit.fused_done = False
                armed += 1
        return armed

    @torch.no_grad()
    def step(self, closure: Callable[[], Tensor] | None = None, *, grad_scale: Tensor | None = None) -> Tensor | None:  # type: ignore[override]
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        _refresh_status_guard(self.param_groups)
        for group in self.param_groups:
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            lr = float(lr)
            units: dict[int, Any] = {}
            unit_members: dict[int, int] = {}
            plain: list[Tensor] = []
            for p in group["params"]:
                unit = getattr(p, "_fs2_unit", None)
                if unit is not None:
                    units[id(unit)] = unit
                    unit_members[id(unit)] = unit_members.get(id(unit), 0) + 1
                    self._init_state(p)
                elif p.grad is not None:
                    plain.append(p)
            # ---- flat units: one launch each
            for uid, unit in units.items():
                if getattr(unit, "fused_done", False):
                    # the reduce-scatter of this unit has already applied the update: only the step count moves
                    step = unit.fused_step["step"]
                    unit.fused_step, unit.fused_done = None, False
                    for sp in unit.shard_params:
                        st = self.state[sp]
                        st["_host_step"] = step
                        st["step"].fill_(step)
                    continue
                unit.fused_step = None
                if not unit.grads_ready or unit.grad_shard is None:
                    continue
                if unit_members[uid] != len(unit.shard_params):
                    raise ValueError("All parameters of an FSDP unit must be in the same optimizer parameter group.")
                st0 = self.state[unit.shard_params[0]]
                step = int(st0["step"].item()) + 1 if "_host_step" not in st0 else st0["_host_step"] + 1
                m, v = self._unit_moments(unit)
                offloaded = unit.master.device != unit.low_shard.device
                low = unit.low_shard if (unit.low_shard.dtype == torch.bfloat16 and not offloaded) else None
                grad = unit.grad_shard
                gs = grad_scale
                if offloaded:            # CPU offload: the update runs where the fp32 state lives
                    grad = grad.to(unit.master.device)
                    gs = grad_scale.to(unit.master.device) if grad_scale is not None else None
                # Parameters that received no gradient since ``zero_grad`` (frozen, or unused in this step) are
                # left alone -- no weight decay, no moment decay -- as ``torch.optim.AdamW`` leaves parameters
                # whose ``grad`` is None: one launch per maximal run of adjacent parameters that took part.
                took = getattr(unit, "took_part", None)
                if took is None or all(took):
                    ranges = [(0, unit.shard_size)]
                else:
                    ranges = []
                    for s, t in zip(unit.specs, took):
                        if not t:
                            continue
                        if ranges and ranges[-1][1] == s.shard_off:
                            ranges[-1] = (ranges[-1][0], s.shard_off + s.shard_numel)
                        else:
                            ranges.append((s.shard_off, s.shard_off + s.shard_numel))
                for lo, hi in ranges:
                    multi_tensor_adamw([unit.master[lo:hi]], [grad[lo:hi]], [m[lo:hi]], [v[lo:hi]],
                                       [low[lo:hi] if low is not None else None], lr=lr, beta1=b1, beta2=b2,
                                       eps=eps, weight_decay=wd, step=step, grad_scale=gs)
                if low is None:
                    unit.low_shard.copy_(unit.master, non_blocking=True)
                for sp in unit.shard_params:
                    st = self.state[sp]
                    st["_host_step"] = step
                    st["step"].fill_(step)
            # ---- ordinary parameters
            if plain:
                ms, vs, gs, lows, masters = [], [], [], [], []
                step = 0
                for p in plain:
                    st = self._init_state(p)
                    step = st.get("_host_step", int(st["step"].item())) + 1
                    st["_host_step"] = step
                    st["step"].fill_(step)
                    ms.append(st["exp_avg"])
                    vs.append(st["exp_avg_sq"])
                    gs.append(p.grad)
                if all(p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and p.data_ptr() % 16 == 0
                       and g.is_contiguous() and g.data_ptr() % 16 == 0 for p, g in zip(plain, gs)):
                    multi_tensor_adamw(plain, gs, ms, vs, [None] * len(plain), lr=lr, beta1=b1, beta2=b2, eps=eps,
                                       weight_decay=wd, step=step, grad_scale=grad_scale)
                else:
                    for p, g, m, v in zip(plain, gs, ms, vs):
                        if p.dtype == torch.float32:
                            adamw_reference(p, g, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                                            step=step, grad_scale=grad_scale if grad_scale is not None else 1.0)
                        else:
                            master = self.state[p].setdefault("master", p.detach().float().clone())
                            adamw_reference(master, g, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                                            step=step, grad_scale=grad_scale if grad_scale is not None else 1.0,
                                            low=p)
        return loss

    def state_dict(self) -> dict[str, Any]:  # type: ignore[override]
        for group in self.param_groups:
            for p in group["params"]:
                if getattr(p, "_fs2_unit", None) is not None:
                    self._init_state(p)
        sd = super().state_dict()
        for st in sd["state"].values():
            st.pop("_host_step", None)
        return sd

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:  # type: ignore[override]
        # materialise flat-unit state first so loaded tensors are copied into the flat buffers
        targets: dict[int, dict[str, Tensor]] = {}
        idx = 0
        for group in self.param_groups:
            for p in group["params"]:
                if getattr(p, "_fs2_unit", None) is not None:
                    st = self._init_state(p)
                    targets[idx] = {"exp_avg": st["exp_avg"], "exp_avg_sq": st["exp_avg_sq"]}
                idx += 1
        super().load_state_dict(state_dict)
        idx = 0
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state.get(p)
                if st:
                    if idx in targets:
                        for k in ("exp_avg", "exp_avg_sq"):
                            if st[k].data_ptr() != targets[idx][k].data_ptr():
                                targets[idx][k].copy_(st[k])
                                st[k] = targets[idx][k]
                    if isinstance(st.get("step"), Tensor):
                        st["_host_step"] = int(st["step"].item())
                        st["step"] = st["step"].detach().to("cpu", torch.float32)
                idx += 1
