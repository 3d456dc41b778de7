"""Position encodings."""
from __future__ import annotations

import math

import torch

from ..registry import register_part
from .base import ParamSpec, PositionEncoding, Runtime


def rope_inv_freqs(head_dim: int, theta: float, rotary_dim: int | None = None) -> torch.Tensor:
    """``theta^(-2i/rotary_dim)`` for i < rotary_dim/2 as 32-bit floats
    (src/forward/cpu.rs:1057-1061).  Each entry is computed in double precision and rounded
    once, so the table does not depend on a platform's single-precision ``powf``; the table is
    built on the host and the kernels only index it, as the reference does
    (src/forward/gpu.rs:215-219)."""
    rd = head_dim if rotary_dim is None else rotary_dim
    return torch.tensor([float(theta) ** (-2.0 * i / rd) for i in range(rd // 2)],
                        dtype=torch.float64).to(torch.float32)


class RotaryNeoX(PositionEncoding):
    """Split-half rotary embedding: pair ``(i, i + rotary_dim/2)`` of every query and key head
    is rotated by the 32-bit angle ``position * inv_freq[i]`` (src/forward/cpu.rs:1094-1113)."""

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim must be even and in 2..head_dim, got {self.rotary_dim}")
        self._table: torch.Tensor | None = None

    def rotary(self, rt: Runtime):
        if self._table is None or self._table.device != rt.device:
            self._table = rope_inv_freqs(self.head_dim, self.theta, self.rotary_dim).to(rt.device)
        return self._table, self.rotary_dim


def slowed_long_waves(freqs, factor: float, low: float, high: float, original: float):
    """Frequencies whose long waves are slowed, each in double precision: with wavelength ``L = 2 pi / f``, a wave
    shorter than ``original / high`` keeps f; one longer than ``original / low`` gets ``f / factor``; between the two,
    with ``s = (original / L - low) / (high - low)``, it gets ``(1 - s) f / factor + s f``."""
    out = []
    for f in freqs:
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out.append(f)
        elif wave > original / low:
            out.append(f / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


class RotaryScaledNeoX(RotaryNeoX):
    """Split-half rotary embedding whose table is ``theta^(-2i / rotary_dim)`` with long waves slowed by
    ``slowed_long_waves`` (``scaling``: a dict with ``factor``, ``low``, ``high``, ``original``; None: the plain
    table).  Only the table differs; the kernels index it as any other."""

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None, scaling: dict | None = None):
        super().__init__(head_dim, theta, rotary_dim)
        self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")} if scaling else None

    def rotary(self, rt: Runtime):
        if self._table is None or self._table.device != rt.device:
            f = [self.theta ** (-2.0 * i / self.rotary_dim) for i in range(self.rotary_dim // 2)]
            if self.scaling:
                f = slowed_long_waves(f, **self.scaling)
            self._table = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(rt.device)
        return self._table, self.rotary_dim


class RotaryInterleaved(RotaryNeoX):
    """The same rotation on neighbouring pairs ``(2i, 2i + 1)`` of every head."""

    interleaved = True


class NoPositionEncoding(PositionEncoding):
    """Keys and queries are used as projected."""


class LearnedPositions(PositionEncoding):
    """A learned vector per position, added (unscaled) to the embedded tokens: ``x[t] += table[position[t]]``.
    Positions count from 0 in each request; one beyond the table is an error the step reports."""

    def __init__(self, max_positions: int, hidden_size: int, param: str = "weight"):
        self.n, self.hidden, self.param = int(max_positions), int(hidden_size), str(param)
        self.table: torch.Tensor | None = None

    def param_specs(self):
        return [ParamSpec(self.param, (self.n, self.hidden))]

    def load(self, tensors, rt: Runtime):
        self.table = rt.matrix(tensors[self.param])

    def on_embed(self, x, positions, rt: Runtime) -> None:
        rt.ops.add_rows(x, self.table, positions)


register_part("position", "learned", LearnedPositions)
register_part("position", "rope_neox", RotaryNeoX)
register_part("position", "rope_scaled_neox", RotaryScaledNeoX)
register_part("position", "rope_interleaved", RotaryInterleaved)
register_part("position", "none", NoPositionEncoding)
