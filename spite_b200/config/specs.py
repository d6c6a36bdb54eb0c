"""Plain data that describes a model to the engine.

An architecture's configuration turns itself into a `ModelPlan`: which parts
each layer is made of (by registered kind name and parameters), in which order
the layers run, and which cache each run of a layer uses.  The engine builds
and runs a plan without knowing which architecture produced it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


class ConfigError(ValueError):
    """A configuration that cannot describe a runnable model."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered kind and the constructor's parameters."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items()))))


@dataclass(frozen=True)
class BlockSpec:
    """A layer: how its parts are arranged (`arrangement` is a registered block kind) and the
    parts themselves by the names the arrangement gives its places (`prenorm_residual`:
    mixer_norm, mixer, ffn_norm, ffn).  Another arrangement has other places: more norms, no
    feed-forward, two mixers."""
    arrangement: str
    parts: dict[str, PartSpec] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.arrangement, tuple(sorted((k, hash(v)) for k, v in self.parts.items()))))

    def __getattr__(self, place):
        """`spec.mixer` reads the part at the place `mixer`."""
        parts = self.__dict__.get("parts", {})
        if place in parts:
            return parts[place]
        raise AttributeError(f"block {self.__dict__.get('arrangement')!r} has no place {place!r}; it has {sorted(parts)}")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    `layer` indexes `ModelPlan.blocks` (a layer may be named more than once: its
    weights are then shared).  `cache` names the cache this run uses; two runs
    with the same `cache` read the same keys and values, and only the runs with
    `write_cache` append to it.
    """
    layer: int
    cache: int
    write_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    blocks: tuple[BlockSpec, ...]
    order: tuple[LayerCall, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_positions: int
    embedding_scale: float = 1.0          # the embedding row is multiplied by this as it enters the residual stream
    logit_scale: float = 1.0              # logits are multiplied by this,
    logit_softcap: float | None = None    # then squashed to cap * tanh(logit / cap)

    def validate(self):
        if self.hidden_size <= 0 or self.vocab_size <= 0:
            raise ConfigError("hidden_size and vocab_size must be positive")
        if not self.blocks:
            raise ConfigError("a model needs at least one layer")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        writers = {}
        for call in self.order:
            if not 0 <= call.layer < len(self.blocks):
                raise ConfigError(f"run order names layer {call.layer}, model has {len(self.blocks)}")
            if call.write_cache:
                if call.cache in writers:
                    raise ConfigError(f"cache {call.cache} is written by two runs of the order")
                writers[call.cache] = call.layer
        seen = set()
        for call in self.order:
            if not call.write_cache and call.cache not in seen:
                raise ConfigError(f"cache {call.cache} is read before any run writes it")
            if call.write_cache:
                seen.add(call.cache)
        return self
