"""Stand-in for torcheval's metric classes (metric bookkeeping only; not on the
model / FSDP / optimizer path of the benchmark arm)."""
import torch


class Metric:
    def __init__(self, *, device=None):
        self._device = device

    def to(self, device):
        self._device = device
        return self

    def reset(self):
        return self

    def state_dict(self):
        return {}

    def load_state_dict(self, sd, strict=True):
        pass


class _Agg(Metric):
    def __init__(self, *, device=None):
        super().__init__(device=device)
        self.value = torch.zeros((), device=device, dtype=torch.float64)

    def compute(self):
        return self.value


class Sum(_Agg):
    def update(self, x, *, weight=1.0):
        self.value = self.value + torch.as_tensor(x, device=self._device).sum() * weight
        return self


class Mean(_Agg):
    def __init__(self, *, device=None):
        super().__init__(device=device)
        self.weight = torch.zeros((), device=device, dtype=torch.float64)

    def update(self, x, *, weight=1.0):
        self.value = self.value + torch.as_tensor(x, device=self._device).sum() * weight
        self.weight = self.weight + weight
        return self

    def compute(self):
        return self.value / self.weight.clamp(min=1e-12)


class Max(_Agg):
    def update(self, x):
        self.value = torch.maximum(self.value, torch.as_tensor(x, device=self._device).max().double())
        return self


class Min(_Agg):
    def update(self, x):
        self.value = torch.minimum(self.value, torch.as_tensor(x, device=self._device).min().double())
        return self


class Throughput(_Agg):
    def update(self, n, elapsed):
        return self
