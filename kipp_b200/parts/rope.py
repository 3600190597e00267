"""Rotary position encoding with half-split pairs (src/kipp.c:2368-2382):
pair (i, i + rot/2) of a head is rotated by position * theta^(-2i/rot)."""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
    """``rotary_dim`` leading dims of each head are rotated (all of them by
    default); ``theta`` is the frequency base."""
    kind = "rotary"

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")

    def frequencies(self) -> torch.Tensor:
        """float32 theta^(-2i/rot) for i < rot/2, as the reference's
        powf(theta, -(2.0f * i) / rot): a float32 exponent, the power rounded
        to float32 once (the library computes the same values)."""
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float32)
        exponent = (-(2.0 * i) / float(self.rotary_dim)).double()
        theta = torch.tensor(self.theta, dtype=torch.float32).double()
        return torch.pow(theta, exponent).float()

    def table_key(self):
        return ("rotary", self.theta, self.rotary_dim)

    def describe(self, prefix, ctx) -> dict:
        if self.rotary_dim == 0:
            return {"kind": "no_position"}
        return {"kind": "rotary", "head_dim": self.head_dim, "theta": self.theta, "rotary_dim": self.rotary_dim}


class NoPositionEncoding(PositionEncoding):
    rotary_dim = 0

    def inv_freq(self, device=None):
        return None


class StretchedRotaryEncoding(RotaryEncoding):
    """Rotary frequencies whose long wavelengths are stretched (the frequency
    scaling of Llama 3.1): with l = 2 pi / f, f stays where l < original / high,
    becomes f / factor where l > original / low, and is blended in between."""
    kind = "stretched_rotary"

    def __init__(self, head_dim: int, theta: float, factor: float, low: float, high: float, original: float,
                 rotary_dim: Optional[int] = None):
        super().__init__(head_dim, theta, rotary_dim)
        self.factor, self.low, self.high, self.original = float(factor), float(low), float(high), float(original)

    def frequencies(self) -> torch.Tensor:
        import math
        out = []
        for i in range(self.rotary_dim // 2):
            f = self.theta ** (-2.0 * i / self.rotary_dim)
            wave = 2.0 * math.pi / f
            if wave > self.original / self.low:
                f /= self.factor
            elif not wave < self.original / self.high:
                s = (self.original / wave - self.low) / (self.high - self.low)
                f = (1.0 - s) * f / self.factor + s * f
            out.append(f)
        return torch.tensor(out, dtype=torch.float64).float()

    def table_key(self):
        return ("stretched", self.theta, self.rotary_dim, self.factor, self.low, self.high, self.original)

    def describe(self, prefix, ctx) -> dict:
        return {"kind": "stretched_rotary", "head_dim": self.head_dim, "theta": self.theta, "rotary_dim": self.rotary_dim,
                "factor": self.factor, "low": self.low, "high": self.high, "original": self.original}


class YarnRotaryEncoding(RotaryEncoding):
    """Rotary frequencies scaled by a ramp over the pair index: with
    pair(t) = dims ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(pair(fast)), 0),
    hi = min(ceil(pair(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    the frequency of pair i is f_i / factor * ramp_i + f_i (1 - ramp_i); cos and sin
    are both multiplied by 0.1 ln(factor) + 1."""
    kind = "yarn_rotary"

    def __init__(self, head_dim: int, theta: float, factor: float, original: float, fast: float, slow: float,
                 rotary_dim: Optional[int] = None):
        super().__init__(head_dim, theta, rotary_dim)
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)

    def magnitude(self) -> float:
        import math
        return 0.1 * math.log(self.factor) + 1.0

    def frequencies(self) -> torch.Tensor:
        import math
        dims = self.rotary_dim
        pair = lambda t: dims * math.log(self.original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))   # noqa: E731
        lo, hi = max(math.floor(pair(self.fast)), 0), min(math.ceil(pair(self.slow)), dims - 1)
        out = []
        for i in range(dims // 2):
            f = self.theta ** (-2.0 * i / dims)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / self.factor * ramp + f * (1.0 - ramp))
        return torch.tensor(out, dtype=torch.float64).float()

    def table_key(self):
        return ("yarn", self.theta, self.rotary_dim, self.factor, self.original, self.fast, self.slow)

    def describe(self, prefix, ctx) -> dict:
        return {"kind": "yarn_rotary", "head_dim": self.head_dim, "theta": self.theta, "rotary_dim": self.rotary_dim,
                "factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
