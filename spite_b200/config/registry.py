"""One registry from an architecture's name (config.json `architectures[0]`) to
its configuration class.  A configuration class knows how to read its own
config.json keys, how to describe the model as a `ModelPlan`, and which
checkpoint tensors bind to which parameter of the plan.

Counterpart in giveen/spite: `ArchRegistry` (crates/spite-models/src/lib.rs:386-436),
a list of (architecture string, constructor) with an error for unknown names.
"""
from __future__ import annotations

import json
from pathlib import Path

from .specs import ConfigError

_ARCHITECTURES: dict[str, type] = {}
_MODEL_TYPES: dict[str, str] = {}       # config.json `model_type` -> architecture name, for files without `architectures`


def register_architecture(*names: str, model_types: tuple = ()):
    """Class decorator: `@register_architecture("FooForCausalLM", model_types=("foo",))`."""
    def deco(cls):
        for n in names:
            _ARCHITECTURES[n] = cls
        for t in model_types:
            _MODEL_TYPES[t] = names[0]
        return cls
    return deco


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}") from None


def config_from_dict(d: dict):
    archs = d.get("architectures")
    if isinstance(archs, str):
        archs = [archs]
    if not archs or not isinstance(archs, (list, tuple)):
        name = _MODEL_TYPES.get(d.get("model_type"))
        if name is None:
            raise ConfigError("config.json has no `architectures` list (and no known `model_type`); known architectures: "
                              + (", ".join(known_architectures()) or "(none)"))
        return config_class_for(name).from_dict(d)
    return config_class_for(archs[0]).from_dict(d)


def load_config(folder):
    """Read `<folder>/config.json` and return the typed configuration it names."""
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} not found")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    return config_from_dict(d)
