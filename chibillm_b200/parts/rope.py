"""Position encodings as parts.

"rope": split-half rotation of the first ``rotary_dim`` features of each head,
``inv_freq[j] = theta ** (-2j / rotary_dim)`` computed once in 32-bit on the
host, angle = float(position) * inv_freq[j] in 32-bit
(src/metal/metal_kernels.mm:186-191, src/metal/kernels/tensor_ops.metal:168-197).
The attention kernels apply it themselves from the table (``fused_rotation``).

With ``scaling_factor`` the slow frequencies are stretched (see PositionSpec) and
cosines and sines carry an amplitude other than one; the frequencies are then made
in 64-bit on the host and rounded once.  Kernels that rotate from ``inv_freq`` alone
do not know the amplitude: a mixer asks ``amplitude`` and takes a kernel that does.

"none": no position information inside the mixer.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, Runtime, register_position


def rotary_inverse_frequencies(theta: float, rotary_dim: int) -> torch.Tensor:
    """The table shared by every user of one (theta, rotary_dim): float32 pow of
    float32 arguments, exponent -2j / rotary_dim."""
    j = torch.arange(rotary_dim // 2, dtype=torch.float32)
    exponent = (-2.0 * j) / float(rotary_dim)
    return torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)


def stretched_inverse_frequencies(spec) -> torch.Tensor:
    """The frequencies of a rotation whose slow part is divided by ``scaling_factor``:
    pairs that turn more than ``fast_turns`` times within ``original_positions`` keep
    their frequency, pairs that turn less than ``slow_turns`` times get all of the
    factor, a linear ramp over the pair index lies between."""
    n, theta = spec.rotary_dim, float(spec.theta)
    j = torch.arange(n // 2, dtype=torch.float64)
    freq = theta ** (-2.0 * j / n)

    def pair_that_turns(times: float) -> float:
        return n * math.log(spec.original_positions / (2.0 * math.pi * times)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_that_turns(spec.fast_turns)), 0)
    hi = min(math.ceil(pair_that_turns(spec.slow_turns)), n - 1)
    ramp = ((j - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return (freq * (ramp / float(spec.scaling_factor) + (1.0 - ramp))).to(torch.float32)


def banded_inverse_frequencies(spec) -> torch.Tensor:
    """The frequencies of a rotation scaled by wavelength (PositionSpec.wavelength_bands): short
    waves keep their frequency, long ones are divided by the factor, the band between is blended.
    Made in 64-bit on the host and rounded once."""
    factor, low, high, original = (float(v) for v in spec.wavelength_bands)
    n, theta = spec.rotary_dim, float(spec.theta)
    out = []
    for j in range(n // 2):
        f = theta ** (-2.0 * j / n)
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out.append(f)
        elif wave > original / low:
            out.append(f / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, runtime: Runtime):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and within head_dim {spec.head_dim}")
        self.spec = spec
        self.runtime = runtime
        self.amplitude = 1.0
        bands = getattr(spec, "wavelength_bands", None)
        if bands is not None:
            if spec.scaling_factor:
                raise ValueError("a rotation is stretched either by turns (scaling_factor) or by wavelength bands")
            if len(bands) != 4 or min(bands) <= 0 or bands[1] == bands[2]:
                raise ValueError("wavelength bands need positive factor, low, high, original and low != high")
            self.inv_freq = banded_inverse_frequencies(spec).to(runtime.device)
        elif spec.scaling_factor:
            if spec.scaling_factor <= 0 or spec.original_positions <= 0 or spec.fast_turns <= 0 or spec.slow_turns <= 0:
                raise ValueError("a stretched rotation needs positive factor, original positions and turn counts")
            self.inv_freq = stretched_inverse_frequencies(spec).to(runtime.device)
            self.amplitude = float(spec.amplitude_slope) * math.log(float(spec.scaling_factor)) + 1.0
        else:
            self.inv_freq = rotary_inverse_frequencies(spec.theta, spec.rotary_dim).to(runtime.device)

    def fused_rotation(self):
        return self.inv_freq, self.spec.rotary_dim

    def step_table(self, ctx):
        table_of = getattr(self.runtime.kernels, "rope_table", None)
        if table_of is None:
            return None
        if self.amplitude != 1.0:
            return None                      # the table's readers rotate with amplitude one
        s = self.spec
        key = ("rope", float(s.theta), int(s.rotary_dim), float(s.scaling_factor), int(s.original_positions),
               float(s.fast_turns), float(s.slow_turns), tuple(getattr(s, "wavelength_bands", None) or ()))
        table = ctx.shared.get(key)
        if table is None:
            table = ctx.workspace.get("rope.table." + ".".join(str(v) for v in key[1:]),
                                      (ctx.num_tokens, self.spec.rotary_dim),
                                      torch.float32)
            table_of(ctx.positions, self.inv_freq, self.spec.rotary_dim, table)
            ctx.shared[key] = table
        return table


class NoPosition(PositionEncoding):
    amplitude = 1.0

    def __init__(self, spec, runtime: Runtime):
        self.spec = spec

    def fused_rotation(self):
        return None, 0

    def apply(self, q, k, ctx) -> None:
        return None


register_position("rope", RotaryEncoding, replace=True)
register_position("none", NoPosition, replace=True)
