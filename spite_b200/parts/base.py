"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a `PartSpec` (registered kind + parameters), declares its
parameters and what it needs of the cache, receives its tensors in `bind`, and
runs on the tokens of a step.  No part knows which model it is in: sizes and
constants arrive as constructor parameters.

Kinds of parts and what each must provide:

  norm           `forward(h, out, rows=None)`: out = norm(h[rows]) (h float32)
  position       `frequencies(device)`: rotation frequencies or None
  mixer          `cache_request()`, `forward(x, h, batch, cache)`: adds its output into h
  feed_forward   `forward(x, h, batch)`: adds its output into h
  block          `forward(h, batch, cache)`: one layer on the residual stream h

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


class PositionEncoding(Part):
    def frequencies(self) -> Optional[torch.Tensor]:
        """float32 [head_dim / 2] rotation frequencies on the device, or None for no rotation."""
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
    def forward(self, h, batch, cache):
        raise NotImplementedError
