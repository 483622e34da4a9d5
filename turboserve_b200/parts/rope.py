"""Rotary position encoding (NeoX halves): the constants; the rotation itself runs fused
with the bias add and the cache append in ``layer_ops.cu`` (``PositionEncoding.apply``).

``inv_freq[i] = 1 / theta^(2i / rotary_dim)`` in float32, ``angle = (float32(pos) / factor) *
inv_freq[i]``, the pair ``(i, i + rotary_dim / 2)`` is rotated by it, as
``src/turboserve/engine/model/layers.py:258-302`` builds its tables (``:214-222`` for the
halves). The reference casts cos and sin to the model dtype before the multiply; here angles,
cos, sin and the rotation are fp32 and the result is rounded once.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import PositionEncoding, register_position


class RotaryPosition(PositionEncoding):
    def __init__(self, spec: PartSpec, device: torch.device | str) -> None:
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.factor = float(spec.get("factor", 1.0))
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be even and >= 2, got {self.rotary_dim}")
        if self.theta <= 0 or self.factor <= 0:
            raise ValueError("rope theta and factor must be positive")
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(device)


def scaled_rotary_frequencies(dims: int, base: float, scaling: dict | None = None) -> tuple[torch.Tensor, float]:
    """Frequencies of the pairs ``(i, i + dims / 2)`` and the factor on cos and sin, with YaRN scaling if asked.

    ``f_i = base^(-2i / dims)``. With ``scaling = {factor, original, fast, slow}``: a pair that turns ``t`` times
    over ``original`` positions has index ``d(t) = dims ln(original / (2 pi t)) / (2 ln base)``; between
    ``lo = max(floor(d(fast)), 0)`` and ``hi = min(ceil(d(slow)), dims - 1)`` a ramp
    ``r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` blends ``f_i`` (fast pairs, kept) into ``f_i / factor``
    (slow pairs, stretched): ``f_i / factor * r_i + f_i (1 - r_i)``; cos and sin are multiplied by
    ``0.1 ln(factor) + 1``. Computed in float64 and rounded to float32 once (the angles are float32 products).
    """
    import math

    if dims < 2 or dims % 2:
        raise ValueError(f"rotary dims must be even and >= 2, got {dims}")
    index = torch.arange(dims // 2, dtype=torch.float64)
    freq = float(base) ** (-2.0 * index / dims)
    amplitude = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def pair_index(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

        lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
        hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
        ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        freq = freq / factor * ramp + freq * (1.0 - ramp)
        amplitude = 0.1 * math.log(factor) + 1.0
    return freq.to(torch.float32), amplitude


def wavelength_scaled_frequencies(dims: int, base: float, scaling: dict | None = None) -> torch.Tensor:
    """Frequencies ``f_i = base^(-2i / dims)`` of ``dims / 2`` pairs, long waves stretched by their wavelength.

    With ``scaling = {factor, low, high, original}`` and ``l_i = 2 pi / f_i``: a wave shorter than ``original / high``
    is kept, one longer than ``original / low`` turns ``factor`` times slower (``f_i / factor``), and between the two
    ``s = (original / l_i - low) / (high - low)`` blends them, ``(1 - s) f_i / factor + s f_i``. Computed in
    float64 and rounded to float32 once (the angles are float32 products).
    """
    import math

    if dims < 2 or dims % 2:
        raise ValueError(f"rotary dims must be even and >= 2, got {dims}")
    freq = float(base) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    if scaling:
        factor, low, high, original = (float(scaling[key]) for key in ("factor", "low", "high", "original"))
        if not (factor > 0.0 and high > low and original > 0.0):
            raise ValueError("frequency scaling needs factor > 0, high > low and original > 0")
        wave = 2.0 * math.pi / freq
        blend = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
        mixed = (1.0 - blend) * freq / factor + blend * freq
        freq = torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, mixed))
    return freq.to(torch.float32)


def rotary_frequencies(dims: int, base: float, scaling: dict | None = None) -> tuple[torch.Tensor, float]:
    """Frequencies and the factor on cos and sin for either way of scaling: ``{factor, original, fast, slow}``
    (:func:`scaled_rotary_frequencies`) or ``{factor, low, high, original}`` (:func:`wavelength_scaled_frequencies`)."""
    if scaling and "low" in scaling and "high" in scaling:
        return wavelength_scaled_frequencies(dims, base, scaling), 1.0
    return scaled_rotary_frequencies(dims, base, scaling)


class NoPosition(PositionEncoding):
    """No position encoding: queries and keys are used as projected (bias and append only)."""

    def __init__(self, spec: PartSpec | None = None, device: torch.device | str | None = None) -> None:
        pass


register_position("rotary", RotaryPosition)
register_position("none", NoPosition)
