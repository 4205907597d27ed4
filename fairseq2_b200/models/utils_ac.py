"""Layer-wise activation checkpointing (cf. fairseq2 ``models/utils/ac.py:16-23``)."""
from __future__ import annotations

from typing import Any

import torch
from torch.nn import Module
from torch.utils.checkpoint import checkpoint


class CheckpointWrapper(Module):
    """Recomputes the wrapped layer in backward (non-reentrant, RNG state preserved)."""

    def __init__(self, module: Module) -> None:
        super().__init__()
        self.module = module

    def forward(self, *args: Any, **kwargs: Any) -> Any:
        if not torch.is_grad_enabled():
            return self.module(*args, **kwargs)
        return checkpoint(self.module, *args, use_reentrant=False, preserve_rng_state=True, **kwargs)


def apply_layerwise_ac(model: Module, every_nth_layer: int = 1) -> None:
    """Wraps every n-th element of each ``layers`` ModuleList; parameter names are unchanged in state dicts
    because the wrapper re-exports them through ``state_dict`` hooks of the data-parallel facade."""
    for m in model.modules():
        layers = getattr(m, "layers", None)
        if isinstance(layers, torch.nn.ModuleList):
            for i in range(len(layers)):
                if (i + 1) % every_nth_layer == 0 and not isinstance(layers[i], CheckpointWrapper):
                    inner = layers[i]
                    fwd = inner.forward

                    def make(f):  # type: ignore[no-untyped-def]
                        def wrapped(*a: Any, **kw: Any) -> Any:
                            if not torch.is_grad_enabled():
                                return f(*a, **kw)
                            return checkpoint(f, *a, use_reentrant=False, preserve_rng_state=True, **kw)
                        return wrapped

                    # patch forward in place: keeps module names, FSDP units and hooks intact
                    inner.forward = make(fwd)  # type: ignore[method-assign]
