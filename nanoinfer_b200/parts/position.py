"""Rotary position encoding (half-split / "neox" pairing) as a table of cos and sin.

``inv_freq_i = theta^(-2i/dim)``, ``angle = position * inv_freq_i``; element d < dim/2 pairs with
d + dim/2. Angles are computed in 64-bit and stored as 32-bit cos/sin, as the reference's engine
does (cpp/src/ops.cpp:121-144); its Python oracle computes them in 32-bit
(nanoinfer/layers.py:78-97), which differs by about 1e-4 at position 4096.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import PositionEncoding, Runtime
from .spec import PartSpec


def rotary_tables(max_positions: int, dim: int, theta: float):
    """``(cos, sin)`` of shape ``[max_positions, dim/2]`` in float32, angles in float64."""
    half = dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / float(dim))
    pos = torch.arange(max_positions, dtype=torch.float64)
    ang = torch.outer(pos, inv_freq)
    return ang.cos().to(torch.float32), ang.sin().to(torch.float32)


class RotaryEncoding(PositionEncoding):
    """params: ``dim`` (rotated width of a head), ``theta``, ``max_positions``. No tensors."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(dim: int, theta: float, max_positions: int) -> PartSpec:
        return PartSpec("rotary", {"dim": dim, "theta": theta, "max_positions": max_positions})

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.dim = int(spec.params["dim"])
        if self.dim <= 0 or self.dim % 2:
            raise ValueError(f"rotary dim must be positive and even, got {self.dim}")
        self.max_positions = int(spec.params["max_positions"])
        cos, sin = rotary_tables(self.max_positions, self.dim, float(spec.params["theta"]))
        self.cos = cos.to(rt.device).contiguous()
        self.sin = sin.to(rt.device).contiguous()

    def rotary(self):
        return self.cos, self.sin, self.dim


class NoPositionEncoding(PositionEncoding):
    """Mixers bound to this encoding use their inputs as they are."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec() -> PartSpec:
        return PartSpec("no_position")


register_part("rotary", RotaryEncoding)
register_part("no_position", NoPositionEncoding)


def scaled_frequencies(dims: int, base: float, scaling=None):
    """Frequencies of the ``dims/2`` rotated pairs, ``f_i = base^(-2i/dims)``, optionally rescaled the YaRN way, and
    the factor on cos and sin. ``scaling`` = {factor} alone: every frequency is divided by ``factor`` (linear scaling of
    the positions), cos and sin as they are. ``scaling`` = {factor, original, fast, slow}: a pair that turns more than ``fast``
    times within ``original`` positions keeps its frequency, one that turns fewer than ``slow`` times has it divided
    by ``factor``, linearly blended in between over the pair index: with
    ``turn_dim(t) = dims * ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(turn_dim(fast)), 0)``,
    ``hi = min(ceil(turn_dim(slow)), dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the
    frequency is ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and cos and sin are multiplied by
    ``0.1 ln(factor) + 1``. Computed in 64-bit, returned as (float64 tensor, float)."""
    import math
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / float(dims))
    if not scaling:
        return f, 1.0
    if "original" not in scaling:
        return f / float(scaling["factor"]), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class FrequencyRotary(PositionEncoding):
    """Rotary positions given as a vector of frequencies instead of tables: the kernels form
    ``angle = position * frequency`` in 32-bit themselves, for any position, and rotate pairs in the ``layout``
    "interleaved" (element 2i with 2i + 1; the default) or "half" (i with i + dims/2). params: ``dims`` (rotated width),
    ``base``, ``scaling`` (None or a dict of ``scaled_frequencies``), ``layout``. No tensors. ``rotary()`` is None: mixers
    that want tables cannot bind to it."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(dims: int, base: float, scaling=None, layout: str = "interleaved") -> PartSpec:
        params = {"dims": dims, "base": base, "scaling": dict(scaling) if scaling else None}
        if layout != "interleaved":
            params["layout"] = layout
        return PartSpec("frequency_rotary", params)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.dims = int(spec.params["dims"])
        if self.dims <= 0 or self.dims % 2:
            raise ValueError(f"rotated width must be positive and even, got {self.dims}")
        self.layout = str(spec.params.get("layout", "interleaved"))
        if self.layout not in ("interleaved", "half"):
            raise ValueError(f"unknown layout of rotated pairs '{self.layout}'")
        f, self.magnitude = scaled_frequencies(self.dims, float(spec.params["base"]), spec.params.get("scaling"))
        self.freq = f.to(torch.float32).to(rt.device).contiguous()

    def frequencies(self):
        """(frequencies [dims/2] float32 on the device, factor on cos and sin, dims)."""
        return self.freq, self.magnitude, self.dims


register_part("frequency_rotary", FrequencyRotary)
