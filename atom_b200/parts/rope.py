"""Rotary position encoding, half-split pairing ("neox"), as
atom/model_ops/rotary_embedding.py:14-24 (rotation) and :58-80 (table):
   inv_freq_j = 1 / theta^(2j / rotary_dim),  angle = pos * inv_freq_j  (32-bit),
   y1 = x1 cos - x2 sin,  y2 = x2 cos + x1 sin  with x1 = x[:d/2], x2 = x[d/2:].
The table stays in 32-bit in both precisions (the reference casts it to the model type,
:49-50); the rotation itself happens inside the mixer's fused kernel."""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, Runtime
from .registry import register


@register("position", "rope_neox")
class RotaryNeox(PositionEncoding):
    graph_safe = True

    def __init__(self, rotary_dim: int, theta: float, max_position: int):
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        self.rotary_dim, self.theta, self.max_position = rotary_dim, theta, max_position
        self._table: Optional[torch.Tensor] = None

    def table(self, rt: Runtime) -> torch.Tensor:
        """[max_position, rotary_dim] float32: cos of every pair's angle, then sin."""
        if self._table is None or self._table.device != rt.device:
            d = self.rotary_dim
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
            t = torch.arange(self.max_position, dtype=torch.float32)
            ang = torch.outer(t, inv_freq)
            self._table = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous().to(rt.device)
        return self._table


def yarn_frequencies(rotary_dim: int, theta: float, factor: float, original: float, fast: float, slow: float):
    """Frequencies of the rotary pairs stretched for sequences longer than ``original`` positions (YaRN, Peng et al.
    2023), and the factor on cos and sin.  With f_i = theta^(-2i / d) and pair(n) = d ln(original / (2 pi n)) /
    (2 ln theta) the pair whose wave makes n turns over the original length: pairs below lo = floor(pair(fast)) keep
    f_i, pairs above hi = ceil(pair(slow)) get f_i / factor, and between them the two are blended linearly.
    Computed in 64-bit."""
    import math

    half = rotary_dim // 2
    f = [theta ** (-2.0 * i / rotary_dim) for i in range(half)]

    def pair(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair(fast)), 0)
    hi = min(math.ceil(pair(slow)), rotary_dim - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@register("position", "rope_yarn")
class RotaryYarn(PositionEncoding):
    """Half-split rotary pairs whose angle is computed in the kernel, position * frequency in 32-bit, from a vector
    of frequencies (so no table bounds the positions), with YaRN's stretch when ``scaling`` is given as
    {factor, original, fast, slow}.  A mixer asks for ``frequencies(rt)`` and ``magnitude`` and hands them to its
    kernel; ``table`` gives None."""
    graph_safe = True

    def __init__(self, rotary_dim: int, theta: float, scaling: Optional[dict] = None):
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        self.rotary_dim, self.theta = rotary_dim, float(theta)
        if scaling:
            self._f, self.magnitude = yarn_frequencies(rotary_dim, self.theta, float(scaling["factor"]),
                                                       float(scaling["original"]), float(scaling["fast"]),
                                                       float(scaling["slow"]))
        else:
            self._f, self.magnitude = [self.theta ** (-2.0 * i / rotary_dim) for i in range(rotary_dim // 2)], 1.0
        self._dev: Optional[torch.Tensor] = None

    def frequencies(self, rt: Runtime) -> torch.Tensor:
        """[rotary_dim / 2] float32 on the device (at least one element, so that it always has an address)."""
        if self._dev is None or self._dev.device != rt.device:
            self._dev = torch.tensor(self._f or [0.0], dtype=torch.float64).to(torch.float32).to(rt.device)
        return self._dev

    def apply(self, q, k, step) -> None:
        raise NotImplementedError("rope_yarn is applied by mixers that take frequencies (latent_attention)")


def wavelength_frequencies(rotary_dim: int, theta: float, factor: float, original: float, low: float, high: float):
    """Frequencies of the rotary pairs stretched by wavelength (the scaling of Llama 3.1): with f_i = theta^(-2i / d) and
    wavelength l = 2 pi / f_i, a pair keeps f_i where l < original / high, takes f_i / factor where l > original / low,
    and between the two blends them with s = (original / l - low) / (high - low): (1 - s) f_i / factor + s f_i.
    Computed in 64-bit."""
    import math

    out = []
    for i in range(rotary_dim // 2):
        f = theta ** (-2.0 * i / rotary_dim)
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out.append(f)
        elif wave > original / low:
            out.append(f / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


@register("position", "rope_wavelength")
class RotaryWavelength(RotaryYarn):
    """As ``rope_yarn`` (angles position * frequency computed in the kernel, no table), with the frequencies stretched by
    wavelength when ``scaling`` is given as {factor, original, low, high}; cos and sin keep their magnitude."""
    graph_safe = True

    def __init__(self, rotary_dim: int, theta: float, scaling: Optional[dict] = None):
        super().__init__(rotary_dim, theta, None)
        if scaling:
            if float(scaling["high"]) == float(scaling["low"]):
                raise ValueError("rope_wavelength: 'high' and 'low' must differ")
            self._f = wavelength_frequencies(rotary_dim, self.theta, float(scaling["factor"]), float(scaling["original"]),
                                             float(scaling["low"]), float(scaling["high"]))


@register("position", "none")
class NoPosition(PositionEncoding):
    graph_safe = True

    def __init__(self):
        pass
