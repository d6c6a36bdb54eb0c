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
