"""Position encodings.  A position part says how q and k are to be rotated (the
frequencies, which elements of a head pair up, how many of them rotate); the
rotation itself runs inside the mixer's prepare kernel, and keys are cached after
it (crates/spite-models/src/llama/llama4.rs:155-186), so the cache and the
attention kernel are the same for every encoding of this kind.
"""
from __future__ import annotations

import math

import torch

from ..config.specs import ConfigError
from .base import PositionEncoding, Rotation, register_position


def rotary_frequencies(head_dim: int, theta: float, scaling: dict | None) -> list[float]:
    """freq_i = theta^(-2i/head_dim) (crates/spite-rope/src/lib.rs:78-82), optionally
    rescaled by the llama3 rule: wavelengths above original/low_freq_factor are divided
    by `factor`, those below original/high_freq_factor are kept, the band between is
    blended linearly (an empty band, high == low, has nothing to blend)."""
    half = head_dim // 2
    freqs = [theta ** (-2.0 * i / head_dim) for i in range(half)]
    if not scaling:
        return freqs
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out.append(f)
        elif wavelen > orig / low:
            out.append(f / factor)
        else:
            s = (orig / wavelen - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


@register_position("rotary_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotation of neighbouring pairs (2i, 2i+1) of every head of q and k."""
    graph_safe = True

    def __init__(self, ctx, head_dim: int, theta: float, scaling: dict | None = None):
        super().__init__(ctx)
        if head_dim % 2:
            raise ConfigError("rotary encoding needs an even head_dim")
        f = rotary_frequencies(int(head_dim), float(theta), scaling)
        self._rotation = Rotation(torch.tensor(f, dtype=torch.float64).to(torch.float32).to(ctx.device), "neighbours")

    def rotation(self):
        return self._rotation


@register_position("no_position")
class NoPosition(PositionEncoding):
    graph_safe = True
    def __init__(self, ctx):
        super().__init__(ctx)

    def rotation(self):
        return None


def yarn_frequencies(rotary_dim: int, theta: float, scaling: dict | None):
    """(frequencies, amplitude) of a rotation whose long wavelengths are stretched (the YaRN rule).

    f_i = theta^(-2i/dims).  With `scaling` = {factor, original, fast, slow}: the pair index at which a
    wavelength makes t turns over the original context is dim(t) = dims ln(original / (2 pi t)) / (2 ln theta);
    lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims - 1); pairs below lo keep f_i, pairs above hi get
    f_i / factor, between them the two are blended linearly in the pair index (an empty band is guarded by a
    width of at least 0.001).  The amplitude 0.1 ln(factor) + 1 multiplies cos and sin."""
    half = rotary_dim // 2
    freqs = [theta ** (-2.0 * i / rotary_dim) for i in range(half)]
    if not scaling:
        return freqs, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return rotary_dim * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), rotary_dim - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@register_position("rotary_yarn")
class RotaryYarn(PositionEncoding):
    """Rotation of neighbouring pairs (2i, 2i+1) of the first `rotary_dim` elements, wavelengths stretched by
    `scaling` (None: the plain frequencies, amplitude one)."""
    graph_safe = True

    def __init__(self, ctx, rotary_dim: int, theta: float, scaling: dict | None = None):
        super().__init__(ctx)
        if rotary_dim % 2 or rotary_dim < 2:
            raise ConfigError("a rotation needs an even number of elements")
        f, amplitude = yarn_frequencies(int(rotary_dim), float(theta), scaling)
        self._rotation = Rotation(torch.tensor(f, dtype=torch.float64).to(torch.float32).to(ctx.device), "neighbours",
                                  int(rotary_dim), float(amplitude))

    def rotation(self):
        return self._rotation


@register_position("rotary_halves")
class RotaryHalves(PositionEncoding):
    """Rotation of the first `rotary_dim` elements of every head of q and k, element i paired with element
    i + rotary_dim / 2; the other elements pass unchanged.  f_i = theta^(-2i / rotary_dim), optionally rescaled by
    wavelength as `rotary_frequencies` describes, with `scaling` = {factor, low, high, original}."""
    graph_safe = True

    def __init__(self, ctx, rotary_dim: int, theta: float, scaling: dict | None = None):
        super().__init__(ctx)
        if rotary_dim % 2 or rotary_dim < 2:
            raise ConfigError("a rotation needs an even number of elements")
        if scaling:
            missing = [k for k in ("factor", "low", "high", "original") if k not in scaling]
            if missing:
                raise ConfigError(f"rotation scaling lacks {missing}")
            scaling = {"factor": scaling["factor"], "low_freq_factor": scaling["low"], "high_freq_factor": scaling["high"],
                       "original_max_position_embeddings": scaling["original"]}
        f = rotary_frequencies(int(rotary_dim), float(theta), scaling)
        self._rotation = Rotation(torch.tensor(f, dtype=torch.float64).to(torch.float32).to(ctx.device), "halves",
                                  int(rotary_dim))

    def rotation(self):
        return self._rotation
