"""Position encodings.  An attention mixer asks its position part for the table of
per-pair inverse frequencies that its fused norm+rotation kernel applies (rotary()); a
part that returns None adds no position information.  Any half-split rotation — scaled
or per-pair adjusted frequencies, a rotation of only the first n_rot dimensions — is a
part that returns its own table.

RotaryNeox: pairs (i, i + n_rot/2); angle = position * theta^(-2i/n_rot), the product
rounded to 32 bits, then sin and cos (imparo-cpu/src/ops.rs:551-569).  The per-pair
inverse frequency is computed in 64-bit on the host and kept as a 32-bit table."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import Part


class PositionEncoding(Part):
    # which dimensions make a rotation pair: False (i, i + n_rot/2), True (2i, 2i + 1)
    interleaved = False
    # a factor on every sine and cosine (1: a pure rotation)
    magnitude = 1.0

    def rotary(self) -> Optional[Tuple[torch.Tensor, int]]:
        """(inv_freq float32 [n_rot/2] on the device, n_rot): dimension i < n_rot/2 pairs
        with i + n_rot/2 and turns by position * inv_freq[i].  None: no rotation."""
        return None


class NoPosition(PositionEncoding):
    pass


class RotaryNeox(PositionEncoding):
    """params: head_dim, theta, n_rot (default head_dim), wavelength_scaling (optional: factor, low, high, original).

    With wavelength_scaling a pair's frequency f depends on its wavelength l = 2 pi / f: kept where l < original / high,
    f / factor where l > original / low, and between the two (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low).  Computed in 64-bit on the host, kept as a 32-bit table."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.head_dim = int(params["head_dim"])
        self.n_rot = int(params.get("n_rot", self.head_dim))
        self.theta = float(params["theta"])
        if self.n_rot % 2 or self.n_rot > self.head_dim:
            raise ValueError(f"rotary: n_rot {self.n_rot} must be even and at most the head size {self.head_dim}")
        i = torch.arange(self.n_rot // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / max(self.n_rot, 1))
        sc = params.get("wavelength_scaling")
        if sc:
            import math
            factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / inv
            s = (original / wavelength - low) / (high - low)
            blended = (1.0 - s) * inv / factor + s * inv
            inv = torch.where(wavelength < original / high, inv, torch.where(wavelength > original / low, inv / factor, blended))
        self.inv_freq = inv.to(torch.float32).to(rt.device)

    def rotary(self):
        return (self.inv_freq, self.n_rot) if self.n_rot else None


class RotaryInterleaved(PositionEncoding):
    """Rotation of the pairs (2i, 2i+1) over the first n_rot dimensions of a head, the rest passing unchanged;
    frequency of pair i: theta^(-2i/n_rot).

    params: head_dim, theta, n_rot (default head_dim), scaling (optional: factor, original, fast, slow).
    With scaling, frequencies are blended between the plain one and the plain one divided by `factor`, by how many
    turns a pair makes over `original` positions: with dim(t) = n_rot * ln(original / (2 pi t)) / (2 ln theta),
    lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), n_rot - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i * (1 - ramp_i);
    and sines and cosines are multiplied by 0.1 * ln(factor) + 1.  The table is computed in 64-bit on the host and
    kept in 32-bit; angles are position * frequency in 32-bit."""
    interleaved = True

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.head_dim = int(params["head_dim"])
        self.n_rot = int(params.get("n_rot", self.head_dim))
        self.theta = float(params["theta"])
        if self.n_rot % 2 or not 0 <= self.n_rot <= self.head_dim:
            raise ValueError(f"rotary: n_rot {self.n_rot} must be even and at most the head size {self.head_dim}")
        self.inv_freq, self.magnitude = self.table(self.n_rot, self.theta, params.get("scaling"))
        self.inv_freq = self.inv_freq.to(torch.float32).to(rt.device)

    @staticmethod
    def table(n_rot: int, theta: float, scaling=None):
        """(frequencies float64 [n_rot/2], magnitude)."""
        import math
        i = torch.arange(n_rot // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * i / max(n_rot, 1))
        if not scaling:
            return f, 1.0
        factor, original = float(scaling["factor"]), float(scaling["original"])
        where = lambda turns: n_rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
        lo = max(math.floor(where(float(scaling["fast"]))), 0)
        hi = min(math.ceil(where(float(scaling["slow"]))), n_rot - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def rotary(self):
        return (self.inv_freq, self.n_rot) if self.n_rot else None
