"""Rotary position encoding.

Reference formula (models/rope.py:14-35): ``inv_freq[j] = 1 / base**(2j/dim)`` for
``j < dim/2`` (32-bit), ``theta = pos * inv_freq[j]`` (32-bit), and the rotation of
**interleaved pairs**: ``out[2j] = x[2j]*cos - x[2j+1]*sin``,
``out[2j+1] = x[2j]*sin + x[2j+1]*cos``.  The reference's CUDA rope kernel rotates
half-split pairs ``(j, j+dim/2)`` instead (kernels/rope_kernel/rope_kernel.cu:133-157);
its serving path and its golden generation use the interleaved form, which is the
default here, and ``style="half"`` gives the other.  The base is fixed in the
reference (models/rope.py:6); here it is this part's parameter.

``inv_freq`` is built once with the reference's own expression so that the angle
``float(pos) * inv_freq[j]`` has the very same 32-bit rounding; the kernels take
sine and cosine of that product in 32-bit.

``scaling`` (optional; ``factor``, ``low``, ``high``, ``original``) rescales the frequencies by their wavelength
``l = 2 pi / f`` against a context length ``original``: a frequency with ``l < original / high`` stays, one with
``l > original / low`` becomes ``f / factor``, and between the two ``s = (original / l - low) / (high - low)`` blends
``(1 - s) f / factor + s f``.  ``dim`` is the number of rotated values; a mixer may rotate only the first ``dim``
values of a wider head.

``scaling`` with ``kind: "yarn"`` (``factor``, ``original``, ``fast``, ``slow``) is YaRN's rescaling by pair index instead:
with ``turn(t) = dim * ln(original / (2 pi t)) / (2 ln base)`` - the (fractional) pair index whose frequency makes ``t`` turns
over ``original`` positions -, ``lo = max(floor(turn(fast)), 0)``, ``hi = min(ceil(turn(slow)), dim - 1)`` and
``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair ``i`` turns at ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``; and
cosine and sine are both multiplied by ``YARN_MAGNITUDE_SLOPE * ln(factor) + 1`` (so a product of two rotated vectors grows by
its square).
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from ..registry import register_part

ROTARY_STYLES = {"interleaved": 0, "half": 1}
YARN_MAGNITUDE_SLOPE = 0.1


@register_part("position", "rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, prefix: str, dim: int, base: float, style: str = "interleaved", scaling=None):
        super().__init__(prefix)
        if dim % 2:
            raise ValueError(f"rotary dimension {dim} must be even (models/rope.py:8)")
        if style not in ROTARY_STYLES:
            raise ValueError(f"unknown rotary style {style!r}; known: {sorted(ROTARY_STYLES)}")
        self.dim, self.base, self.style = int(dim), float(base), style
        self.scaling = None
        self.yarn = None
        if scaling is not None and scaling.get("kind") == "yarn":
            missing = [k for k in ("factor", "original", "fast", "slow") if k not in scaling]
            if missing:
                raise ValueError(f"yarn scaling lacks {missing}")
            self.yarn = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if min(self.yarn.values()) <= 0 or self.base == 1.0:
                raise ValueError(f"yarn scaling {scaling!r}: needs positive constants and a base other than 1")
        elif scaling is not None:
            missing = [k for k in ("factor", "low", "high", "original") if k not in scaling]
            if missing:
                raise ValueError(f"rotary scaling lacks {missing}")
            self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
            if not self.scaling["high"] > self.scaling["low"] or self.scaling["factor"] <= 0 or self.scaling["low"] <= 0:
                raise ValueError(f"rotary scaling {scaling!r}: needs factor > 0 and high > low > 0")
        self._inv_freq = None

    def frequencies(self) -> torch.Tensor:
        """float32 [dim / 2]: the rotation frequency of every pair."""
        if self.yarn is not None:
            y, out = self.yarn, []

            def turn(t):
                return self.dim * math.log(y["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(self.base))

            lo, hi = max(math.floor(turn(y["fast"])), 0), min(math.ceil(turn(y["slow"])), self.dim - 1)
            for i in range(self.dim // 2):                           # few values, once: in 64-bit, rounded at the end
                f = self.base ** (-2.0 * i / self.dim)
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                out.append(f / y["factor"] * ramp + f * (1.0 - ramp))
            return torch.tensor(out, dtype=torch.float64).to(torch.float32)
        if self.scaling is None:
            return 1.0 / (self.base ** (torch.arange(0, self.dim, 2).float() / self.dim))
        sc, out = self.scaling, []
        for i in range(self.dim // 2):                               # few values, once: in 64-bit, rounded at the end
            f = self.base ** (-2.0 * i / self.dim)
            wavelength = 2.0 * math.pi / f
            if wavelength < sc["original"] / sc["high"]:
                out.append(f)
            elif wavelength > sc["original"] / sc["low"]:
                out.append(f / sc["factor"])
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * f / sc["factor"] + s * f)
        return torch.tensor(out, dtype=torch.float64).to(torch.float32)

    @property
    def magnitude(self) -> float:
        """What cosine and sine are multiplied by: 1 unless the frequencies are YaRN's."""
        return 1.0 if self.yarn is None else YARN_MAGNITUDE_SLOPE * math.log(self.yarn["factor"]) + 1.0

    def bind(self, ops, dtype, device):
        super().bind(ops, dtype, device)
        self._inv_freq = self.frequencies().to(device=device, dtype=torch.float32).contiguous()

    def rotary_table(self):
        return self._inv_freq, ROTARY_STYLES[self.style]

    def step_table(self, ctx):
        """cos/sin of every token of the step, computed once per step and shared by all layers whose
        encoding has the same dimension and base (kept in the step's context)."""
        if not hasattr(self.ops, "rope_table"):
            return None
        tables = ctx.step_cache
        key = ("rope_table", self.dim, self.base, None if self.scaling is None else tuple(sorted(self.scaling.items())),
               None if self.yarn is None else tuple(sorted(self.yarn.items())))
        if key not in tables:
            if self.yarn is None:
                tables[key] = self.ops.rope_table(ctx.positions, self._inv_freq)
            else:
                tables[key] = self.ops.rope_table(ctx.positions, self._inv_freq, self.magnitude)
        return tables[key]

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary encoding runs inside the fused rotate-and-store kernel")


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No position encoding: keys and queries are stored and used as projected."""

    def __init__(self, prefix: str = ""):
        super().__init__(prefix)

    def rotary_table(self):
        return None, 0

    def step_table(self, ctx):
        return None

    def apply(self, q, k, positions):
        return None
