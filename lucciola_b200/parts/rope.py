"""Rotary position encoding, half-rotation ("NeoX") pairing: for i < rot/2 the pair
(x[i], x[i + rot/2]) is rotated by pos * theta^(-2i/rot) (src/kernels/rope.cu:28-60 of lucciola,
where theta is the literal 1e6 at src/qwen.cc:636; here it is a parameter).

The table of inverse frequencies is made once on the host in float32; the kernel forms the
angle as one float32 product pos * inv_freq[i].

With `yarn` = (factor, original, fast, slow) the frequencies are scaled for contexts beyond the `original` positions
(YaRN): with turns(t) = rot * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turns(fast)), 0),
hi = min(ceil(turns(slow)), rot - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns by
f_i / factor * ramp_i + f_i * (1 - ramp_i): pairs that turn fast keep their frequency, slow ones are divided by the
factor.  Sines and cosines are multiplied by `magnitude` = 0.1 ln(factor) + 1.  That table is made in float64 and
rounded once."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from .base import PositionEncoding, Runtime


class RotaryEmbedding(PositionEncoding):
    recordable = True

    def __init__(self, rt: Runtime, head_dim: int, theta: float, rot_dim: int | None = None,
                 yarn: Optional[Sequence[float]] = None):
        self.rt = rt
        self.head_dim = head_dim
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rotary size {self.rot_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        exponent = torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / float(self.rot_dim)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)
        self.magnitude = 1.0                 # factor on the rotation's sines and cosines
        if yarn is not None:
            inv, self.magnitude = yarn_frequencies(self.rot_dim, self.theta, *yarn)
        self.inv_freq = inv.to(rt.device)

    def rotary_table(self):
        return self.inv_freq, self.rot_dim


def yarn_frequencies(rot_dim: int, theta: float, factor: float, original: float, fast: float, slow: float) -> tuple[torch.Tensor, float]:
    """(float32 frequencies [rot_dim / 2], magnitude) of a rotation with YaRN scaling (see the module's text)."""
    i = torch.arange(rot_dim // 2, dtype=torch.float64)
    f = float(theta) ** (-2.0 * i / rot_dim)
    turns = lambda t: rot_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))
    lo = max(math.floor(turns(fast)), 0)
    hi = min(math.ceil(turns(slow)), rot_dim - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0
