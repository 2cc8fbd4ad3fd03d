"""Rotary position encoding: the table of inverse frequencies."""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .base import PositionEncoding, Runtime, register_position


def rotary_inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> List[float]:
    """freq_j = theta^(-2j / rotary_dim) for j < rotary_dim / 2, in float64
    (ExiledOfCode/KuiperLLama builds sin/cos tables from 1 / pow(theta, d / head_size) with
    theta fixed per build, rope_kernel.cu:38-49,124-135; here theta is a parameter).

    ``scaling`` with rope_type "llama3" rescales by wavelength 2 pi / freq: shorter than
    original / high_freq_factor unchanged; longer than original / low_freq_factor divided
    by factor; between them interpolated linearly in original / wavelength.  rope_type "linear" divides every
    frequency by ``factor``; "yarn" is ``yarn_frequencies``.  KuiperLLama has
    no such rule; this follows the published meaning of those config.json keys."""
    freqs = [1.0 / (float(theta) ** ((2.0 * j) / rotary_dim)) for j in range(rotary_dim // 2)]
    if scaling is None:
        return freqs
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return freqs
    if kind == "yarn":
        return yarn_frequencies(freqs, rotary_dim, float(theta), scaling)
    if kind == "linear":                               # positions stretched by a factor: every frequency divided by it
        return [f / float(scaling["factor"]) for f in freqs]
    if kind != "llama3":
        raise ValueError(f"unknown rope scaling {kind!r}")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < orig / high:
            out.append(f)
        elif wavelength > orig / low:
            out.append(f / factor)
        else:
            smooth = (orig / wavelength - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


def yarn_frequencies(freqs: List[float], rotary_dim: int, theta: float, scaling: dict) -> List[float]:
    """The "yarn" rule: pairs that turn fast keep their frequency, pairs that turn slowly have it divided by
    ``factor``, with a linear ramp over the pair index between.  The ramp's ends are the (fractional) pair
    indices whose wave makes ``fast`` and ``slow`` turns in ``original`` positions,
    index(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta), rounded outwards and kept inside the
    pairs; a ramp shorter than 0.001 is taken as that long."""
    factor, orig = float(scaling["factor"]), float(scaling["original"])
    index = lambda turns: rotary_dim * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index(float(scaling["slow"]))), rotary_dim - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out


def rotary_magnitude(scaling: Optional[dict]) -> float:
    """The factor on cos and sin: 1, or with "yarn" scaling ``magnitude_slope`` * ln(factor) + 1."""
    if scaling is None or scaling.get("rope_type", scaling.get("type")) != "yarn":
        return 1.0
    return float(scaling.get("magnitude_slope", 0.1)) * math.log(float(scaling["factor"])) + 1.0


@register_position("rope")
class RotaryPosition(PositionEncoding):
    """Spec: ``head_dim``, ``theta``, ``scaling`` (None, a llama3 dict, a yarn dict or a linear dict) and optionally
    ``rotary_dim`` (default: the whole head) and ``pairing`` ("half": element i with i + rotary_dim / 2, the
    default; "interleaved": element 2i with 2i + 1).  The rotation itself happens in the mixer's kernels;
    this part owns the frequencies, the factor on cos and sin (``magnitude``) and the pairing."""

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        freqs = rotary_inverse_frequencies(self.rotary_dim, float(spec["theta"]), spec.get("scaling"))
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.magnitude = rotary_magnitude(spec.get("scaling"))
        self.pairing = str(spec.get("pairing") or "half")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown pairing {self.pairing!r} (half, interleaved)")

    def rotary(self):
        return self.inv_freq, self.rotary_dim
