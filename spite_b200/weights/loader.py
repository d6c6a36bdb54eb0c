"""Bind checkpoint tensors to a plan's parameters by tensor name.

Everything is checked before anything is copied: one `WeightError` lists every
missing tensor, every tensor of the wrong shape and every tensor the model does
not know.  giveen/spite fails lazily, at the first forward that asks for an
absent tensor (crates/spite-models/src/dense.rs:67-71) and reports wrong shapes
as matvec errors (dense.rs:226-233); the eager check here is deliberate.

Storage rule: floating tensors are kept in bfloat16 (float16 is converted), a
tensor the file stores in 32-bit floats stays 32-bit, integer tables become int32.

A binding may name a layout transform that turns the checkpoint's tensor into the
parameter (the stacked experts are stored input-major and are transposed, for
instance).  Transforms are registered by name; another architecture adds its own
with `register_weight_transform` (a permutation of rows, a slice of a fused tensor).
"""
from __future__ import annotations

import torch

from .safetensors_io import SafetensorsError, open_checkpoint


class WeightError(ValueError):
    def __init__(self, folder, missing, wrong_shape, unexpected, other=()):
        self.missing = list(missing)
        self.wrong_shape = list(wrong_shape)
        self.unexpected = list(unexpected)
        self.other = list(other)
        lines = [f"checkpoint {folder} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += [f"    {n} {list(s)}" for n, s in self.missing]
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += [f"    {n}: file has {list(got)}, model needs {list(want)}" for n, got, want in self.wrong_shape]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += [f"    {n}" for n in self.unexpected]
        for o in self.other:
            lines.append(f"  {o}")
        super().__init__("\n".join(lines))


_TRANSFORMS: dict = {}


def register_weight_transform(name: str):
    """Decorator: `fn(tensor) -> tensor` becomes the transform `name` of a `WeightBinding`.  The function
    gets the checkpoint tensor (already in its storage type, on the target device)."""
    def deco(fn):
        _TRANSFORMS[name] = fn
        return fn
    return deco


def weight_transforms() -> list[str]:
    return sorted(_TRANSFORMS)


@register_weight_transform("transpose_last2")
def _transpose_last2(t):
    """[..., in, out] -> [..., out, in]"""
    return t.transpose(-1, -2).contiguous()


def apply_binding(binding, tensor, device="cpu"):
    """The parameter that `binding` makes of the checkpoint tensor `tensor`."""
    t = tensor.to(storage_dtype(tensor.dtype)).to(device)
    if binding.transform is None:
        return t
    try:
        fn = _TRANSFORMS[binding.transform]
    except KeyError:
        raise ValueError(f"unknown weight transform {binding.transform!r} for {binding.source}; "
                         f"registered: {', '.join(weight_transforms())}") from None
    return fn(t)


def bind_tensors(config, source: dict, device="cpu", folder="(tensors in memory)") -> dict[str, torch.Tensor]:
    """The same binding for checkpoint tensors that are already in memory: `source` maps checkpoint
    tensor names (without prefix) to tensors.  One `WeightError` lists what does not fit."""
    bindings = config.weight_bindings()
    missing = [(b.source, b.source_shape) for b in bindings if b.source not in source]
    wrong = [(b.source, tuple(source[b.source].shape), b.source_shape) for b in bindings
             if b.source in source and tuple(source[b.source].shape) != tuple(b.source_shape)]
    used = {b.source for b in bindings}
    unexpected = sorted(n for n in source if n not in used)
    if missing or wrong or unexpected:
        raise WeightError(folder, missing, wrong, unexpected)
    return {b.target: apply_binding(b, source[b.source], device) for b in bindings}


def storage_dtype(file_dtype: torch.dtype) -> torch.dtype:
    if file_dtype in (torch.float32, torch.float64):
        return torch.float32
    if file_dtype.is_floating_point:
        return torch.bfloat16
    return torch.int32


def load_bound_tensors(folder, config, device="cpu") -> dict[str, torch.Tensor]:
    """{parameter name of the plan: tensor on `device`}, shapes `[out, in]`."""
    try:
        files = open_checkpoint(folder)
    except SafetensorsError as e:
        raise WeightError(folder, [], [], [], [str(e)]) from None
    try:
        where = {}
        for f in files:
            for name in f.names():
                where[name] = f
        bindings = config.weight_bindings()
        prefixes = getattr(config, "checkpoint_prefixes", ("",))
        ignored = tuple(getattr(config, "ignored_prefixes", ()))
        # the prefix under which most expected tensors are found
        prefix = max(prefixes, key=lambda p: sum((p + b.source) in where for b in bindings))
        missing, wrong, used = [], [], set()
        for b in bindings:
            name = prefix + b.source
            if name not in where:
                missing.append((name, b.source_shape))
                continue
            used.add(name)
            got = where[name].entries[name][1]
            if tuple(got) != tuple(b.source_shape):
                wrong.append((name, got, b.source_shape))
        unexpected = sorted(n for n in where if n not in used and not n.startswith(ignored))
        if missing or wrong or unexpected:
            raise WeightError(folder, missing, wrong, unexpected)
        out = {}
        for b in bindings:
            name = prefix + b.source
            out[b.target] = apply_binding(b, where[name].tensor(name), device)
        return out
    finally:
        for f in files:
            f.close()
