"""``to_tensor`` helper (cf. ``src/fairseq2/utils/tensor.py``)."""
from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from fairseq2_b200.typing import DataType, Device


def to_tensor(data: Any, dtype: DataType | None = None, device: Device | None = None) -> Tensor:
    if device is None or device.type != "cuda":
        return torch.tensor(data, dtype=dtype, device=device)
    t = torch.tensor(data, dtype=dtype, device="cpu", pin_memory=True)
    return t.to(device, non_blocking=True)
