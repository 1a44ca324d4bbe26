"""Rotary position encoding from an explicit array of positions."""
from __future__ import annotations

import math
from typing import Tuple

import torch

from .. import ops
from ..config.registry import POSITIONS
from ..config.specs import PositionSpec
from .base import PositionEncoding, StepContext


@POSITIONS.register("rope")
class RotaryEmbedding(PositionEncoding):
    """cos/sin of p_t * theta^(-2j/rotary_dim) for the tokens of a step, computed once per
    step and shared by every layer with an equal specification.  The frequency table is
    float64 and carries quadrants per position, as the reference's does
    (pulsar-core/inc/pulsar/rope.hpp:52-69): its relative error is scaled by the position."""

    def __init__(self, spec: PositionSpec):
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and within head_dim {spec.head_dim}")
        if spec.scaling is not None:
            factor, low, high, original = spec.scaling
            if not (factor > 0.0 and original > 0.0 and high > low > 0.0):
                raise ValueError(f"rotary scaling {spec.scaling}: factor and original must be positive and high > low > 0")
        self.spec = spec
        self._table = {}

    def frequency(self, j: int) -> float:
        """Radians per position of pair j: theta^(-2j / rotary_dim), rescaled by its wavelength where the
        specification says so (``PositionSpec.scaling``)."""
        f = self.spec.theta ** (-2.0 * j / self.spec.rotary_dim)
        if self.spec.scaling is None:
            return f
        factor, low, high, original = self.spec.scaling
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            return f
        if wavelength > original / low:
            return f / factor
        blend = (original / wavelength - low) / (high - low)
        return (1.0 - blend) * f / factor + blend * f

    def quadrants_per_position(self, device) -> torch.Tensor:
        t = self._table.get(device)
        if t is None:
            half = self.spec.rotary_dim // 2
            values = [self.frequency(j) * (2.0 / math.pi) for j in range(half)]
            t = torch.tensor(values, dtype=torch.float64).to(device)
            self._table[device] = t
        return t

    def tables(self, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        key = ("rope", self.spec)
        got = ctx.shared.get(key)
        if got is None:
            half = self.spec.rotary_dim // 2
            tag = f"rope.{self.spec.rotary_dim}.{self.spec.theta}.{self.spec.scaling}"
            cos = ctx.scratch(tag + ".cos", (ctx.n_tokens, half), torch.float32)
            sin = ctx.scratch(tag + ".sin", (ctx.n_tokens, half), torch.float32)
            ops.rope_table(ctx.positions, self.quadrants_per_position(ctx.device), cos, sin)
            got = ctx.shared[key] = (cos, sin)
        return got
