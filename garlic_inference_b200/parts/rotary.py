"""Rotary position encoding: the table of angles, or the frequencies alone.

inv_freq[i] = theta^(-2i/r) for i < r/2 and angle = position * inv_freq[i],
scaling 1.0 (src/src-cuda/rope.cu:3-23,41-79; upstream uses the fast
`__powf`/`__sincosf`, which lose accuracy at large positions).  `rotary_dim`
r may be smaller than the head (the rest of the head passes through).

Parameters beyond upstream's:
  * `layout`: "half" pairs dimension i with i + r/2 (upstream's); "interleaved"
    pairs dimension 2i with 2i + 1.  The mixer's kernel does the rotation; this
    part only says which.
  * `yarn` = {factor, original, fast, slow}: YaRN scaling of the frequencies.
    With dim(t) = r ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(dim(fast)), 0),
    hi = min(ceil(dim(slow)), r - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    pair i turns with f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin
    are both multiplied by 0.1 ln(factor) + 1 (`magnitude`).
  * `linear_factor` s: position interpolation, every frequency divided by s (the angles of position p are those
    of p / s without it).
  * `tables`: True (default) builds float32 cos and sin [max_positions, r/2]
    on the host in float64; False builds none, for models without a limit on
    positions: the mixer's kernel then makes the angle as the float32 product
    position * frequency and takes its cosine and sine itself.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_part


class RotaryPositions(PositionEncoding):
    kind = "rotary"
    graph_safe = True

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        self.layout = params.get("layout", "half")
        self.yarn = params.get("yarn")
        self.linear_factor = float(params.get("linear_factor", 1.0))
        if not self.linear_factor > 0:
            raise ValueError(f"linear_factor must be positive, found {self.linear_factor}")
        if self.layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout {self.layout!r} is neither 'half' nor 'interleaved'")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        freq, self.magnitude = self.frequencies(self.rotary_dim, self.theta, self.yarn, self.linear_factor)
        self.inv_freq = freq.to(torch.float32).to(rt.device)
        self.cos = self.sin = None
        if params.get("tables", True):
            cos, sin = self.build_tables(self.rotary_dim, self.theta, self.max_positions, self.yarn, self.linear_factor)
            self.cos = cos.to(rt.device)
            self.sin = sin.to(rt.device)

    @staticmethod
    def frequencies(rotary_dim: int, theta: float, yarn=None, linear_factor: float = 1.0):
        """(float64 angle per position of each pair [r/2], factor on cos and sin)."""
        i = torch.arange(rotary_dim // 2, dtype=torch.float64)
        f = theta ** (-2.0 * i / rotary_dim) / linear_factor
        if not yarn:
            return f, 1.0
        factor, original = float(yarn["factor"]), float(yarn["original"])

        def dim_of(turns: float) -> float:
            return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

        lo = max(math.floor(dim_of(float(yarn["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(yarn["slow"]))), rotary_dim - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    @staticmethod
    def build_tables(rotary_dim: int, theta: float, max_positions: int, yarn=None, linear_factor: float = 1.0):
        f, mag = RotaryPositions.frequencies(rotary_dim, theta, yarn, linear_factor)
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * f[None, :]
        return (ang.cos() * mag).to(torch.float32).contiguous(), (ang.sin() * mag).to(torch.float32).contiguous()

    def rotary_tables(self):
        if self.cos is None:
            return None
        if self.layout != "half":
            raise ValueError("rotary tables are read by kernels of the 'half' layout only")
        return self.cos, self.sin, self.rotary_dim

    def rotary_frequencies(self):
        """(float32 frequencies [r/2] on the device, factor on cos and sin, r, layout) for kernels that make
        their angles from the position."""
        return self.inv_freq, self.magnitude, self.rotary_dim, self.layout


register_part(RotaryPositions.kind, RotaryPositions)
