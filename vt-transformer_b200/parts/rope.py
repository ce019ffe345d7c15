"""Position encodings of attention: the rotation of pairs, or none."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_part


def rotation_table(max_positions: int, dim: int, base: float) -> torch.Tensor:
    """[max_positions, dim / 2, 2] of (cos, sin) in float32, built as vt-transformer builds
    its table (v1/tensortype/common.cpp:6-24): inv_freq[i] = 1 / pow(base, 2i / dim) in
    double, rounded to float; the angle is the float product position * inv_freq; cos and
    sin of that angle.  The pairing (i, i + dim/2) is the kernel's
    (v1/tensortype/cuda_kernels/rotary_embed.cu:19-29)."""
    base32 = torch.tensor(base, dtype=torch.float32).item()
    inv = torch.tensor([1.0 / math.pow(base32, (2.0 * i) / dim) for i in range(dim // 2)],
                       dtype=torch.float64).to(torch.float32)
    pos = torch.arange(max_positions, dtype=torch.float32)
    angle = (pos[:, None] * inv[None, :]).to(torch.float64)
    return torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).contiguous()


@register_part("position", "rotary")
class RotaryEmbedding(PositionEncoding):
    """Holds the (cos, sin) table on the device; one table for all layers of equal
    (dim, base, max_positions)."""

    _tables = {}

    def load(self, get) -> None:
        key = (self.spec.dim, float(self.spec.base), self.spec.max_positions, str(self.rt.device))
        table = RotaryEmbedding._tables.get(key)
        if table is None:
            table = rotation_table(self.spec.max_positions, self.spec.dim, self.spec.base).to(self.rt.device)
            RotaryEmbedding._tables[key] = table
        self.table = table


@register_part("position", "none")
class NoPosition(PositionEncoding):
    table = None

    def load(self, get) -> None:
        self.table = None


def rotation_frequencies(dim: int, base: float, scaling=None) -> torch.Tensor:
    """[dim / 2] float32: base^(-2i/dim), formed in double and rounded once.  ``scaling`` = (factor, low, high,
    original): a frequency f with wavelength l = 2 pi / f stays where l < original / high, becomes f / factor where
    l > original / low, and between the two (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    out = []
    for i in range(dim // 2):
        f = math.pow(float(base), -2.0 * i / dim)
        if scaling is not None:
            factor, low, high, original = (float(v) for v in scaling)
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


@register_part("position", "rotary_computed")
class ComputedRotary(PositionEncoding):
    """The rotation of the first ``dim`` dimensions of a head, pairs (i, i + dim/2), by the angle
    position * base^(-2i/dim): the kernel that rotates forms the angle as a 32-bit product and takes its cos and sin
    there, so there is no table and no limit of positions.  Holds the [dim/2] frequencies on the device.  With a
    ``ramp`` the frequencies are those of ``ramped_frequencies`` and cos and sin are multiplied by ``mult``."""

    table = None
    mult = 1.0

    def load(self, get) -> None:
        self.frequencies, self.mult = None, 1.0
        if not self.spec.dim:
            return
        if self.spec.ramp is not None:
            if self.spec.scaling is not None:
                raise ValueError("rotary_computed: either 'scaling' or 'ramp'")
            f, self.mult = ramped_frequencies(self.spec.dim, self.spec.base, self.spec.ramp)
            self.frequencies = f.to(self.rt.device)
        else:
            self.frequencies = rotation_frequencies(self.spec.dim, self.spec.base, self.spec.scaling).to(self.rt.device)


def ramped_frequencies(dim: int, base: float, ramp=None):
    """([dim / 2] float32, m): f_i = base^(-2i/dim) in double, rounded once.  ``ramp`` = (factor, original, fast, slow): with
    n(t) = dim ln(original / (2 pi t)) / (2 ln base), lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dim - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns with f_i / factor * r_i + f_i (1 - r_i), and
    m = 0.1 ln(factor) + 1 multiplies cos and sin (1 without a ramp)."""
    f = [math.pow(float(base), -2.0 * i / dim) for i in range(dim // 2)]
    mult = 1.0
    if ramp is not None:
        factor, original, fast, slow = (float(v) for v in ramp)

        def pair_of(turns: float) -> float:
            return dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), dim - 1)
        for i in range(len(f)):
            r = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            f[i] = f[i] / factor * r + f[i] * (1.0 - r)
        mult = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=torch.float64).to(torch.float32), mult


@register_part("position", "rotary_interleaved")
class InterleavedRotary(PositionEncoding):
    """The rotation of the first ``dim`` dimensions of a vector in pairs (2i, 2i + 1), the angle position * f_i formed as a
    32-bit product where it is used, cos and sin multiplied by ``mult``.  Holds the [dim/2] frequencies on the device."""

    table = None

    def load(self, get) -> None:
        self.frequencies, self.mult = None, 1.0
        if self.spec.dim:
            f, self.mult = ramped_frequencies(self.spec.dim, self.spec.base, self.spec.ramp)
            self.frequencies = f.to(self.rt.device)
