"""Position encoders (cf. fairseq2 ``nn/position_encoder.py``: sinusoidal :70,
learned :220, ``RotaryEncoder`` :294, ``ReferenceRotaryEncoder`` :455).

Every encoder takes ``(seqs, seqs_layout, state_bag=None)``; positions come
from ``BatchLayout.position_indices`` so packed, padded and incremental inputs
share one code path. The rotary encoder hands the rotation to the fused kernel
``fairseq2_b200.ops.rope``.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from typing import Callable

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.incremental_state import IncrementalStateBag
from fairseq2_b200.ops.rope import apply_rope
from fairseq2_b200.typing import DataType, Device


class PositionEncoder(Module, ABC):
    def __init__(self, encoding_dim: int) -> None:
        super().__init__()
        self.encoding_dim = encoding_dim

    @abstractmethod
    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor: ...


def _positions(layout: BatchLayout, start: int, *, i32: bool = False) -> Tensor:
    p = layout.position_indices_i32 if i32 else layout.position_indices
    if start:
        p = torch.where(p >= 0, p + start, p)
    return p


def _start_step(module: Module, state_bag: IncrementalStateBag | None) -> int:
    return state_bag.step_nr if (state_bag is not None and not module.training) else 0


def _check_len(layout: BatchLayout, start: int, max_seq_len: int) -> None:
    n = start + layout.max_seq_len
    if n > max_seq_len:
        raise ValueError(
            f"The lengths of all sequences in `seqs` must be less than or equal to the maximum sequence length ({max_seq_len}), but at least one sequence is of length {n} instead.")


def fill_sinusoidal_table(out: Tensor, steps: Tensor, correction: int = 1) -> None:
    """tensor2tensor layout: first half sines, second half cosines."""
    dim = out.shape[-1]
    half = dim // 2
    idx = torch.arange(half, device=steps.device, dtype=torch.float32)
    inv = torch.exp(idx * -math.log(10000.0) / max(half - correction, 1))
    ang = torch.outer(steps.float(), inv)
    out[:, :half] = ang.sin()
    out[:, half:] = ang[:, : dim - half].cos()


class SinusoidalPositionEncoder(PositionEncoder):
    def __init__(self, encoding_dim: int, max_seq_len: int, *, _legacy_pad_idx: int | None = None,
                 device: Device | None = None) -> None:
        super().__init__(encoding_dim)
        if encoding_dim % 2:
            raise ValueError(f"`encoding_dim` must be even, but is {encoding_dim} instead.")
        self.max_seq_len = max_seq_len
        self.sin_offset = 0 if _legacy_pad_idx is None else 1 + _legacy_pad_idx
        self.register_buffer("freqs", torch.empty((max_seq_len, encoding_dim), device=device, dtype=torch.float32),
                             persistent=False)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.reset_non_persistent_buffers()

    def reset_non_persistent_buffers(self) -> None:
        if self.freqs.device.type == "meta":
            return
        steps = torch.arange(self.sin_offset, self.sin_offset + self.max_seq_len, device=self.freqs.device)
        fill_sinusoidal_table(self.freqs, steps)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        start = _start_step(self, state_bag)
        _check_len(seqs_layout, start, self.max_seq_len)
        pos = _positions(seqs_layout, start)
        enc = self.freqs[pos.clamp(min=0)] * (pos >= 0).unsqueeze(-1)
        while enc.ndim < seqs.ndim:
            enc = enc.unsqueeze(-2)
        return (seqs.float() + enc).type_as(seqs)

    def extra_repr(self) -> str:
        return f"encoding_dim={self.encoding_dim}, max_seq_len={self.max_seq_len}"


class LearnedPositionEncoder(PositionEncoder):
    def __init__(self, encoding_dim: int, max_seq_len: int, *, device: Device | None = None,
                 dtype: DataType | None = None) -> None:
        super().__init__(encoding_dim)
        self.max_seq_len = max_seq_len
        self.weight = Parameter(torch.empty((max_seq_len, encoding_dim), device=device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        torch.nn.init.normal_(self.weight)

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        start = _start_step(self, state_bag)
        _check_len(seqs_layout, start, self.max_seq_len)
        pos = _positions(seqs_layout, start)
        enc = torch.nn.functional.embedding(pos.clamp(min=0), self.weight) * (pos >= 0).unsqueeze(-1)
        while enc.ndim < seqs.ndim:
            enc = enc.unsqueeze(-2)
        return seqs + enc.to(seqs.dtype)


class RotaryEncoder(PositionEncoder):
    """Rotates interleaved feature pairs ``(x[2i], x[2i+1])`` by ``pos * theta^(-2i/E)``.

    ``freqs_init_fn(encoder) -> Tensor[E/2]`` may return custom inverse
    frequencies (LLaMA-3.1 smoothing, YaRN). The table is a non-persistent fp32
    buffer ``[max_seq_len, E/2, 2]`` of (cos, sin).
    """

    def __init__(self, encoding_dim: int, max_seq_len: int, *, theta: float = 10_000.0,
                 freqs_init_fn: Callable[["RotaryEncoder"], Tensor] | None = None,
                 device: Device | None = None) -> None:
        super().__init__(encoding_dim)
        if encoding_dim % 2:
            raise ValueError(f"`encoding_dim` must be even, but is {encoding_dim} instead.")
        self.max_seq_len, self.theta, self.freqs_init_fn = max_seq_len, theta, freqs_init_fn
        self.register_buffer("freqs", torch.empty((max_seq_len, encoding_dim // 2, 2), device=device,
                                                  dtype=torch.float32), persistent=False)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.reset_non_persistent_buffers()

    def reset_non_persistent_buffers(self) -> None:
        if self.freqs.device.type == "meta":
            return
        dev = self.freqs.device
        if self.freqs_init_fn is not None:
            inv = self.freqs_init_fn(self).to(device=dev, dtype=torch.float32)
        else:
            idx = torch.arange(0, self.encoding_dim, 2, device=dev, dtype=torch.float32)
            inv = 1.0 / (self.theta ** (idx / self.encoding_dim))
        steps = torch.arange(self.max_seq_len, device=dev, dtype=torch.float32)
        ang = torch.outer(steps, inv)
        self.freqs[..., 0] = ang.cos()
        self.freqs[..., 1] = ang.sin()

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        """``seqs``: ``([N], S, [H], E)``."""
        start = _start_step(self, state_bag)
        _check_len(seqs_layout, start, self.max_seq_len)
        pos = _positions(seqs_layout, start, i32=True)
        lead = pos.ndim
        if seqs.ndim == lead + 1:  # no head dim
            return apply_rope(seqs.unsqueeze(-2), self.freqs, pos).squeeze(-2)
        return apply_rope(seqs, self.freqs, pos)

    def extra_repr(self) -> str:
        return f"encoding_dim={self.encoding_dim}, max_seq_len={self.max_seq_len}, theta={self.theta}"


class DualRotaryEncoder(RotaryEncoder):
    """Rotary encoder with two frequency bands: the first half of the feature dimension rotates with ``theta``,
    the second half with ``dual_theta`` (short- and long-range positions side by side; used by Gemma 3n's LAuReL
    blocks, cf. fairseq2 ``nn/position_encoder.py:928-1009``).

    Both bands live in ONE ``(cos, sin)`` table -- the inverse frequencies of the two half-width encoders laid end
    to end -- so a forward pass is a single rotation over the whole feature dimension instead of two rotations
    and a concatenation.
    """

    def __init__(self, encoding_dim: int, max_seq_len: int, *, theta: float = 10_000.0,
                 dual_theta: float = 100_000.0, device: Device | None = None) -> None:
        if encoding_dim % 4:
            raise ValueError(f"`encoding_dim` must be divisible by 4 for dual RoPE, but is {encoding_dim} instead.")
        self.dual_theta = dual_theta

        def init(enc: RotaryEncoder) -> Tensor:
            half = enc.encoding_dim // 2
            idx = torch.arange(0, half, 2, dtype=torch.float32) / half
            return torch.cat([1.0 / (enc.theta ** idx), 1.0 / (dual_theta ** idx)])

        super().__init__(encoding_dim, max_seq_len, theta=theta, freqs_init_fn=init, device=device)

    def extra_repr(self) -> str:
        return (f"encoding_dim={self.encoding_dim}, max_seq_len={self.max_seq_len}, theta={self.theta}, "
                f"dual_theta={self.dual_theta}")


class ReferenceRotaryEncoder(PositionEncoder):
    """Half-rotation RoPE (``rotate_half`` as in HF/GPT-NeoX): pairs are
    ``(x[i], x[i + E/2])``."""

    def __init__(self, encoding_dim: int, max_seq_len: int, *, theta: float = 10_000.0,
                 device: Device | None = None) -> None:
        super().__init__(encoding_dim)
        if encoding_dim % 2:
            raise ValueError(f"`encoding_dim` must be even, but is {encoding_dim} instead.")
        self.max_seq_len, self.theta = max_seq_len, theta
        self.register_buffer("cos", torch.empty((max_seq_len, encoding_dim), device=device, dtype=torch.float32),
                             persistent=False)
        self.register_buffer("sin", torch.empty((max_seq_len, encoding_dim), device=device, dtype=torch.float32),
                             persistent=False)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.reset_non_persistent_buffers()

    def reset_non_persistent_buffers(self) -> None:
        if self.cos.device.type == "meta":
            return
        dev = self.cos.device
        idx = torch.arange(0, self.encoding_dim, 2, device=dev, dtype=torch.float32)
        inv = 1.0 / (self.theta ** (idx / self.encoding_dim))
        ang = torch.outer(torch.arange(self.max_seq_len, device=dev, dtype=torch.float32), inv)
        ang = torch.cat([ang, ang], dim=-1)
        self.cos.copy_(ang.cos())
        self.sin.copy_(ang.sin())

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout, *, state_bag: IncrementalStateBag | None = None) -> Tensor:
        start = _start_step(self, state_bag)
        _check_len(seqs_layout, start, self.max_seq_len)
        pos = _positions(seqs_layout, start).clamp(min=0)
        cos, sin = self.cos[pos], self.sin[pos]
        while cos.ndim < seqs.ndim:
            cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
        x = seqs.float()
        half = self.encoding_dim // 2
        rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
        return (x * cos + rot * sin).type_as(seqs)


class InterpolatedPositionEncoder(PositionEncoder, ABC):
    """Base of N-d sinusoidal encoders whose grid is resized by interpolation."""


class Sinusoidal2dPositionEncoder(InterpolatedPositionEncoder):
    """Fixed 2-D sin/cos table over an ``(H, W)`` grid, bicubically resized to
    the input grid (ViT/JEPA patch embeddings). Input ``(N, H, W, E)``."""

    def __init__(self, encoding_dim: int, grid_dims: tuple[int, int], *, uniform_power: bool = False,
                 device: Device | None = None) -> None:
        super().__init__(encoding_dim)
        self.grid_dims = grid_dims
        self.uniform_power = uniform_power
        self.register_buffer("freqs", torch.empty((*grid_dims, encoding_dim), device=device, dtype=torch.float32),
                             persistent=False)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.reset_non_persistent_buffers()

    def reset_non_persistent_buffers(self) -> None:
        if self.freqs.device.type == "meta":
            return
        h, w = self.grid_dims
        dev = self.freqs.device
        half = self.encoding_dim // 2
        th = torch.empty((h, half), device=dev)
        tw = torch.empty((w, self.encoding_dim - half), device=dev)
        fill_sinusoidal_table(th, torch.arange(h, device=dev), correction=0)
        fill_sinusoidal_table(tw, torch.arange(w, device=dev), correction=0)
        self.freqs[..., :half] = th[:, None, :]
        self.freqs[..., half:] = tw[None, :, :]

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout | None = None, *, state_bag=None) -> Tensor:  # type: ignore[override]
        h, w = seqs.shape[1:3]
        f = self.freqs
        if (h, w) != self.grid_dims:
            f = torch.nn.functional.interpolate(f.permute(2, 0, 1).unsqueeze(0), size=(h, w), mode="bicubic",
                                                align_corners=False).squeeze(0).permute(1, 2, 0)
        return (seqs.float() + f).type_as(seqs)


class Sinusoidal3dPositionEncoder(InterpolatedPositionEncoder):
    """3-D variant for video patches. Input ``(N, D, H, W, E)``."""

    def __init__(self, encoding_dim: int, grid_dims: tuple[int, int, int], *, uniform_power: bool = False,
                 device: Device | None = None) -> None:
        super().__init__(encoding_dim)
        self.grid_dims = grid_dims
        self.uniform_power = uniform_power
        self.register_buffer("freqs", torch.empty((*grid_dims, encoding_dim), device=device, dtype=torch.float32),
                             persistent=False)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.reset_non_persistent_buffers()

    def reset_non_persistent_buffers(self) -> None:
        if self.freqs.device.type == "meta":
            return
        d, h, w = self.grid_dims
        dev = self.freqs.device
        if self.uniform_power:
            e = int(math.ceil(self.encoding_dim / 6) * 2)
            sizes = [e, e, e]
        else:
            eh = int(math.ceil(self.encoding_dim / 4) * 2)
            sizes = [self.encoding_dim - 2 * eh + 0, eh, eh] if self.encoding_dim - 2 * eh > 0 else [eh, eh, eh]
            sizes = [eh, eh, eh]
        tabs = []
        for n, s in zip((d, h, w), sizes):
            t = torch.empty((n, s), device=dev)
            fill_sinusoidal_table(t, torch.arange(n, device=dev), correction=0)
            tabs.append(t)
        full = torch.cat([
            tabs[0][:, None, None, :].expand(d, h, w, -1),
            tabs[1][None, :, None, :].expand(d, h, w, -1),
            tabs[2][None, None, :, :].expand(d, h, w, -1)], dim=-1)
        self.freqs.copy_(full[..., : self.encoding_dim])

    def forward(self, seqs: Tensor, seqs_layout: BatchLayout | None = None, *, state_bag=None) -> Tensor:  # type: ignore[override]
        dims = tuple(seqs.shape[1:4])
        f = self.freqs
        if dims != self.grid_dims:
            f = torch.nn.functional.interpolate(f.permute(3, 0, 1, 2).unsqueeze(0), size=dims, mode="trilinear",
                                                align_corners=False).squeeze(0).permute(1, 2, 3, 0)
        return (seqs.float() + f).type_as(seqs)
