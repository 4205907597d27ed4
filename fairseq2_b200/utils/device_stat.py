"""Device memory statistics (cf. ``src/fairseq2/utils/device_stat.py``)."""
from __future__ import annotations

from typing import Any

import torch

from fairseq2_b200.typing import Device


class DeviceStatTracker:
    def get_stats(self) -> dict[str, Any]:
        return {}

    def reset_stats(self) -> None:
        pass


class CudaDeviceStatTracker(DeviceStatTracker):
    def __init__(self, device: Device) -> None:
        self._device = device
        self._total = torch.cuda.get_device_properties(device).total_memory

    def get_stats(self) -> dict[str, Any]:
        s = torch.cuda.memory_stats(self._device)
        peak_active = s.get("active_bytes.all.peak", 0)
        peak_reserved = s.get("reserved_bytes.all.peak", 0)
        return {
            "peak_active_mem_bytes": peak_active,
            "peak_active_mem_ratio": peak_active / self._total,
            "peak_reserved_mem_bytes": peak_reserved,
            "peak_reserved_mem_ratio": peak_reserved / self._total,
            "num_alloc_retries": s.get("num_alloc_retries", 0),
            "num_ooms": s.get("num_ooms", 0),
        }

    def reset_stats(self) -> None:
        torch.cuda.reset_peak_memory_stats(self._device)


def create_device_stat_tracker(device: Device) -> DeviceStatTracker:
    if device.type == "cuda":
        return CudaDeviceStatTracker(device)
    return DeviceStatTracker()
