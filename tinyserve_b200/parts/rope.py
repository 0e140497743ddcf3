"""Rotary position encoding: the per-step cos/sin tables.

Formula (upstream src/tinyserve/layers.py:61-65): ``inv_freq[i] = theta ** (-2i / rotary_dim)``
in float64, ``angle = position * inv_freq`` in float64, cos and sin taken in float64 and
rounded to float32. The rotation itself (pairs ``i`` and ``i + rotary_dim/2`` for the "half"
pairing, neighbours ``2i, 2i+1`` for "interleaved"; src/tinyserve/layers.py:84-91 has the
former) is applied by the mixer's fused kernel, which receives these tables. ``scaling``: the four
keys of the rule by wavelength below, or ``{"factor": f}`` alone for linear scaling (every
frequency divided by ``f``).
"""

from __future__ import annotations

import math
from typing import Any

import torch

from ..kernels import ops
from .base import EVERY_STEP, PositionEncoding, Rotation, StepContext, register_position_encoding

RotaryTables = Rotation      # the step's position data of a rotary encoding is the rotation itself


def scale_by_wavelength(freq: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequency scaling by wavelength (the Llama 3.1 rule), in float64: with wavelength
    ``l = 2 pi / f``, ``f`` stays where ``l < original / high``, becomes ``f / factor`` where
    ``l > original / low``, and in between is ``(1 - s) f / factor + s f`` with
    ``s = (original / l - low) / (high - low)``."""
    if not (factor > 0 and high > low and original > 0):
        raise ValueError(f"rotary scaling needs factor > 0, high > low, original > 0; got {factor}, {low}, {high}, {original}")
    wavelength = 2.0 * math.pi / freq
    s = (original / wavelength - low) / (high - low)
    blended = (1.0 - s) * freq / factor + s * freq
    out = torch.where(wavelength > original / low, freq / factor, blended)
    return torch.where(wavelength < original / high, freq, out)


class RotaryEncoding(PositionEncoding):
    recordable = EVERY_STEP

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, pairing: str = "half",
                 scaling: "dict[str, float] | None" = None) -> None:
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim={rotary_dim} must be even and at most head_dim={head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing must be 'half' or 'interleaved', got {pairing!r}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta, self.pairing = float(theta), pairing
        two_i = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        self._inv_freq_host = self.theta ** (-two_i / self.rotary_dim)
        self.scaling = None
        if scaling and set(scaling) == {"factor"}:
            # linear scaling: every frequency divided by the factor (positions stretched by it)
            if not float(scaling["factor"]) > 0:
                raise ValueError(f"rotary scaling factor must be positive, got {scaling['factor']}")
            self.scaling = ("linear", float(scaling["factor"]))
            self._inv_freq_host = self._inv_freq_host / self.scaling[1]
        elif scaling:
            self.scaling = tuple(float(scaling[k]) for k in ("factor", "low", "high", "original"))
            self._inv_freq_host = scale_by_wavelength(self._inv_freq_host, *self.scaling)
        self._inv_freq: torch.Tensor | None = None

    def key(self) -> Any:
        return ("rope", self.rotary_dim, self.theta, self.pairing, self.scaling)

    def prepare(self, ctx: StepContext) -> RotaryTables:
        dev = ctx.positions.device
        if self._inv_freq is None or self._inv_freq.device != dev:
            self._inv_freq = self._inv_freq_host.to(dev)
        half = self.rotary_dim // 2
        cos = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        sin = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        ops.rope_tables(ctx.positions, self._inv_freq, cos, sin)
        return RotaryTables(cos, sin, self.rotary_dim, self.pairing == "interleaved")


register_position_encoding("rope", RotaryEncoding)
