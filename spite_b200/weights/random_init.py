"""Random-weights mode: write a model folder (config.json, model.safetensors)
from a configuration and a seed.

Every tensor is drawn from its own generator, seeded by (seed, tensor name), so
a tensor's values do not depend on which other tensors exist or in which order
they are written.  Norm gains are ones.  Counterpart in giveen/spite: the test
kit that writes a tiny valid GGUF (crates/spite-testkit/src/lib.rs:50-81).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .safetensors_io import save_file


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(seed, name, shape, init, std, dtype, device="cpu"):
    if init == "ones":
        return torch.ones(shape, dtype=dtype, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(tensor_seed(seed, name))
    t = torch.empty(shape, dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=g)
    return t.to(dtype)


def random_checkpoint_tensors(config, seed: int = 0, std: float = 0.02, dtype=torch.bfloat16, device="cpu") -> dict:
    """{checkpoint tensor name: tensor} for `config`, as `write_random_model` would store them (the same
    values on the CPU; another device has its own generator).  For models that are too large to be worth
    writing: `Model.from_tensors` binds them like a checkpoint read from disk."""
    return {b.source: random_tensor(seed, b.source, b.source_shape, b.init, std, dtype, device)
            for b in config.weight_bindings()}


def write_random_model(folder, config, seed: int = 0, std: float = 0.02, dtype=torch.bfloat16):
    """Create `folder` with config.json and model.safetensors for `config`."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_checkpoint_tensors(config, seed, std, dtype)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    save_file(tensors, folder / "model.safetensors", metadata={"format": "pt", "seed": seed, "std": std})
    return folder
