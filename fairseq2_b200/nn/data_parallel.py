"""Uniform facade over "no wrapper" / DDP / FSDP models
(cf. fairseq2 ``nn/data_parallel.py:36-253``): ``state_dict``,
``load_state_dict``, ``no_sync``, ``clip_grad_norm``,
``summon_full_parameters`` plus the hooks a training step needs
(``finish_backward``, ``scale_grads``, ``grad_scale``)."""
from __future__ import annotations

from contextlib import contextmanager, nullcontext
from typing import Any, Iterator, Mapping

import torch
from torch import Tensor
from torch.nn import Module

from fairseq2_b200.nn.utils.grad import clip_grad_norm as _clip_plain
from fairseq2_b200.nn.utils.grad import scale_grads as _scale_plain


class DataParallelFacade:
    """Wraps ``module`` (plain, ``DDP`` or ``FSDP``) behind one interface."""

    def __init__(self, module: Module) -> None:
        from fairseq2_b200.parallel.ddp import DDP
        from fairseq2_b200.parallel.fsdp import FSDP

        self.module = module
        self.kind = "fsdp" if isinstance(module, FSDP) else "ddp" if isinstance(module, DDP) else "none"

    @property
    def base_module(self) -> Module:
        return self.module.module if self.kind != "none" else self.module  # type: ignore[return-value]

    def __call__(self, *a: Any, **kw: Any) -> Any:
        return self.module(*a, **kw)

    def parameters(self):  # type: ignore[no-untyped-def]
        return self.module.parameters()

    def named_parameters(self):  # type: ignore[no-untyped-def]
        return self.module.named_parameters()

    def train(self, mode: bool = True) -> None:
        self.module.train(mode)

    def state_dict(self) -> dict[str, Any]:
        if self.kind == "ddp":
            return self.module.module.state_dict()  # type: ignore[union-attr]
        return self.module.state_dict()

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        if self.kind == "ddp":
            self.module.module.load_state_dict(state_dict)  # type: ignore[union-attr]
        else:
            self.module.load_state_dict(state_dict)

    def no_sync(self):  # type: ignore[no-untyped-def]
        if self.kind == "none":
            return nullcontext()
        return self.module.no_sync()  # type: ignore[operator]

    def zero_grad(self) -> None:
        self.module.zero_grad(set_to_none=True)
        self._plain_scale: Tensor | None = None

    def finish_backward(self) -> None:
        if self.kind != "none":
            self.module.finish_backward()  # type: ignore[operator]

    def scale_grads(self, factor: Tensor | float) -> None:
        if self.kind == "fsdp":
            self.module.scale_grads(factor)  # type: ignore[operator]
        else:
            _scale_plain(self.base_module, factor)

    @property
    def grad_scale(self) -> Tensor | None:
        """Device scalar the optimizer must multiply into the gradients (FSDP
        defers scaling into its fused step); ``None`` if already applied."""
        if self.kind == "fsdp":
            return self.module.grad_scale  # type: ignore[return-value]
        return None

    def clip_grad_norm(self, max_norm: float | None) -> Tensor:
        if self.kind == "fsdp":
            return self.module.clip_grad_norm(max_norm)  # type: ignore[operator]
        return _clip_plain(self.base_module, max_norm)

    def after_optimizer_step(self) -> None:
        if self.kind == "fsdp":
            self.module.after_optimizer_step()  # type: ignore[operator]

    def check_comm_status(self) -> None:
        """Raises ``KernelWaitTimeout`` if a peer-memory collective of this process gave up waiting for a peer.
        Costs one read of a host-mapped word; does not synchronise with the device."""
        check = getattr(self.module, "check_comm_status", None)
        if check is not None:
            check()
            return
        arena = getattr(self.module, "arena", None)
        if arena is not None:
            arena.ext.check_status()

    def summon_full_parameters(self):  # type: ignore[no-untyped-def]
        if self.kind == "fsdp":
            return self.module.summon_full_parameters()  # type: ignore[operator]
        return nullcontext()


def get_data_parallel_facade(module: Module) -> DataParallelFacade:
    return DataParallelFacade(module)
