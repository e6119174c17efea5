"""Rotary position encoding with half-split pairs (i, i + half).

angle = pos / theta^(2i/rotary_dim); src/model/math.rs:52-99.  ``prepare``
fills one cos/sin table per step; every mixer that shares the same
specification reuses it.  A specification with ``scaling`` rescales the
frequencies by their wavelength (see ``rescaled_frequencies``).
"""
from __future__ import annotations

import math

import torch

from ..config.spec import PositionSpec
from ..errors import Unsupported
from ..kernels import ops
from .base import ROTATION, Part, Rotation, register_position_encoding


def rescaled_frequencies(theta: float, rotary_dim: int, scaling) -> list:
    """f_i = theta^(-2i/rotary_dim) for i < rotary_dim / 2, in double precision; with scaling = (factor, low, high,
    original) and wavelength l = 2 pi / f: f where l < original / high, f / factor where l > original / low, and
    between the two (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    out = []
    for i in range(rotary_dim // 2):
        f = theta ** (-2.0 * i / rotary_dim)
        if scaling is not None:
            factor, low, high, original = scaling
            wave = 2.0 * math.pi / f
            if wave > original / low:
                f = f / factor
            elif wave >= original / high:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def ramped_frequencies(theta: float, rotary_dim: int, ramp):
    """-> (frequencies, length).  f_i = theta^(-2i/rotary_dim); with ramp = (factor, original, fast, slow): the pair index at
    which a wave turns n times over ``original`` positions is index(n) = rotary_dim ln(original / (2 pi n)) / (2 ln theta);
    between lo = max(floor(index(fast)), 0) and hi = min(ceil(index(slow)), rotary_dim - 1) the share r_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1) of f_i is divided by the factor: f_i (1 - r_i) + f_i r_i / factor.  The rotated vectors grow
    by length = 0.1 ln(factor) + 1.  Double precision, on the host, once per model."""
    factor, original, fast, slow = ramp
    index = lambda turns: rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(index(fast)), 0)
    hi = min(math.ceil(index(slow)), rotary_dim - 1)
    out = []
    for i in range(rotary_dim // 2):
        f = theta ** (-2.0 * i / rotary_dim)
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


@register_position_encoding("rotary_half")
class RotaryHalf(Part):
    applies = ROTATION

    def __init__(self, spec: PositionSpec, mctx):
        self.spec = spec
        self.half = spec.rotary_dim // 2
        self.key = ("rotary_half", spec.theta, spec.rotary_dim, spec.scaling, spec.ramp)
        self.freq, self.length = None, 1.0
        if spec.scaling is not None and spec.ramp is not None:
            raise Unsupported("a rotary encoding rescales its frequencies by wavelength or along a ramp, not both")
        if spec.scaling is not None:
            self.freq = torch.tensor(rescaled_frequencies(spec.theta, spec.rotary_dim, spec.scaling),
                                     dtype=torch.float64, device=mctx.device)
        if spec.ramp is not None:
            freq, self.length = ramped_frequencies(spec.theta, spec.rotary_dim, spec.ramp)
            self.freq = torch.tensor(freq, dtype=torch.float64, device=mctx.device)

    def rotation(self, ctx) -> Rotation:
        """The rotation of this step's tokens: cos / sin float32 [T, rotary_dim/2], half-split pairs."""
        got = ctx.tables.get(self.key)
        if got is None:
            tag = f"{self.spec.theta}" if self.freq is None else f"{self.spec.theta}.{self.spec.scaling}.{self.spec.ramp}"
            cos = ctx.workspace.get(f"rope.cos.{tag}", ctx.T, self.half, torch.float32)
            sin = ctx.workspace.get(f"rope.sin.{tag}", ctx.T, self.half, torch.float32)
            if self.freq is None:
                ops.rope_table(ctx.positions, cos, sin, self.spec.theta, self.spec.rotary_dim)
            else:
                ops.rope_table_freq(ctx.positions, self.freq, cos, sin, self.length)
            got = ctx.tables[self.key] = Rotation(cos, sin, self.half, interleaved=False)
        return got


@register_position_encoding("rotary_interleaved")
class RotaryInterleaved(RotaryHalf):
    """The same angles, position * theta^(-2i/rotary_dim), applied to the element pairs (2i, 2i + 1)."""

    def __init__(self, spec: PositionSpec, mctx):
        super().__init__(spec, mctx)
        self.key = ("rotary_interleaved", spec.theta, spec.rotary_dim, spec.scaling, spec.ramp)

    def rotation(self, ctx) -> Rotation:
        got = ctx.tables.get(self.key)
        if got is None:
            base = super().rotation(ctx)          # the tables do not depend on which elements form a pair
            got = ctx.tables[self.key] = Rotation(base.cos, base.sin, base.pairs, interleaved=True)
        return got
