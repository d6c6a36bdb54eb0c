"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a `PartSpec` (registered kind + parameters), declares its
parameters and what it needs of the cache, receives its tensors in `bind`, and
runs on the tokens of a step.  No part knows which model it is in: sizes and
constants arrive as constructor parameters.

Kinds of parts and what each must provide:

  norm           `forward(h, out, rows=None)`: out = norm(h[rows]) (h float32)
  position       `rotation()`: a `Rotation` (frequencies, which elements pair up, how many
                 leading elements of a head rotate) or None
  mixer          `cache_request()`, `forward(x, h, batch, cache)`: adds its output into h
  feed_forward   `forward(x, h, batch)`: adds its output into h
  block          `places` (name -> family of each part it is made of),
                 `forward(h, batch, cache)`: one layer on the residual stream h

`h` is the float32 residual stream [M, hidden]; `x` is a normalised copy in the
activation type.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.specs import ConfigError, PartSpec

_REGISTRIES: dict[str, dict[str, type]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {},
}


def _register(family: str, kind: str):
    def deco(cls):
        _REGISTRIES[family][kind] = cls
        cls.kind = kind
        return cls
    return deco


def register_norm(kind):
    return _register("norm", kind)


def register_position(kind):
    return _register("position", kind)


def register_mixer(kind):
    return _register("mixer", kind)


def register_feed_forward(kind):
    return _register("feed_forward", kind)


def register_block(kind):
    return _register("block", kind)


def registered(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])


@dataclass
class BuildContext:
    """What a part may use while it is built and bound."""
    kernels: object            # a KernelSet
    dtype: torch.dtype         # activation and weight type
    device: torch.device


def build_part(family: str, spec: PartSpec, ctx: BuildContext):
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise ConfigError(f"no {family} of kind {spec.kind!r} is registered; known: {', '.join(sorted(reg))}")
    try:
        return reg[spec.kind](ctx, **spec.params)
    except TypeError as e:
        raise ConfigError(f"{family} {spec.kind!r}: bad parameters {sorted(spec.params)} ({e})") from None


@dataclass(frozen=True)
class ParamSpec:
    shape: tuple
    init: str = "normal"       # "normal" | "ones": how random weights fill it


class Part:
    """Common behaviour: parameters by local name."""
    kind = "?"
    #: names of kernel libraries (csrc) the part launches; compiled when a model is built
    kernel_libraries: tuple = ()
    #: the part launches kernels of the kernel set only and never reads device data on the
    #: host, so a step that contains it can be captured in a CUDA graph
    graph_safe = False

    def __init__(self, ctx: BuildContext):
        self.ctx = ctx
        self.k = ctx.kernels

    def param_specs(self) -> dict[str, ParamSpec]:
        return {}

    def bind(self, params: dict[str, torch.Tensor]):
        """Take ownership of the tensors named in `param_specs` (already on the device)."""

    def weight_bytes(self) -> int:
        return 0


class Norm(Part):
    def forward(self, h, out, rows=None):
        raise NotImplementedError


@dataclass(frozen=True)
class Rotation:
    """How a position part wants q and k encoded; the mixer's prepare kernel does it.
    Pair i of a head is rotated by position * inv_freq[i].  `pairing` says which two elements
    pair i is: "neighbours" (2i, 2i+1) or "halves" (i, i + rotary_dim/2).  Only the first
    `rotary_dim` elements of a head rotate (None: all of them)."""
    inv_freq: torch.Tensor              # float32 [rotary_dim / 2] on the device
    pairing: str = "neighbours"
    rotary_dim: Optional[int] = None

    def __post_init__(self):
        if self.pairing not in ("neighbours", "halves"):
            raise ConfigError(f"unknown pairing {self.pairing!r}; use 'neighbours' or 'halves'")


@dataclass(frozen=True)
class QkNorm:
    """RMS norm of every q and k head inside the prepare kernel: after the rotation or before
    it, with gain vectors [head_dim] (float32) or without."""
    eps: float
    before_rotation: bool = False
    q_gain: Optional[torch.Tensor] = None
    k_gain: Optional[torch.Tensor] = None


class PositionEncoding(Part):
    def rotation(self) -> Optional[Rotation]:
        """How q and k are rotated, or None for no rotation."""
        raise NotImplementedError


class Mixer(Part):
    def cache_request(self):
        """(PagedKV | None, FixedState | None): what one cache of this mixer holds."""
        return None, None

    def forward(self, x, h, batch, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, h, batch):
        raise NotImplementedError


class Block(Part):
    """One layer.  An arrangement names its places and the family of the part that fills each
    (`places`); places listed in `optional` may be left out of a `BlockSpec`.  The parts are
    built here and become attributes of the block under their place names."""
    places: dict = {}
    optional: tuple = ()

    def __init__(self, ctx: BuildContext, spec):
        super().__init__(ctx)
        unknown = sorted(set(spec.parts) - set(self.places))
        missing = sorted(n for n in self.places if n not in spec.parts and n not in self.optional)
        if unknown or missing:
            raise ConfigError(f"block {self.kind!r} has the places {sorted(self.places)}: "
                              f"missing {missing}, unknown {unknown}")
        self._children = {}
        for name, family in self.places.items():
            part = build_part(family, spec.parts[name], ctx) if name in spec.parts else None
            setattr(self, name, part)
            if part is not None:
                self._children[name] = part

    def children(self) -> dict:
        """{place: part} of the parts this layer is made of."""
        return dict(self._children)

    def cache_request(self):
        """What one cache of this layer holds: its mixer's request (a layer has at most one
        part that keeps a cache; two such mixers are two layers of the run order)."""
        wants = [c.cache_request() for c in self._children.values() if isinstance(c, Mixer)]
        wants = [w for w in wants if w != (None, None)]
        if len(wants) > 1:
            raise ConfigError(f"block {self.kind!r}: more than one part asks for a cache")
        return wants[0] if wants else (None, None)

    def forward(self, h, batch, cache):
        raise NotImplementedError
