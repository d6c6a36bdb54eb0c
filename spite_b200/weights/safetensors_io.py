"""Reader and writer for the safetensors container: an 8-byte little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw
little-endian tensor bytes.  The reader maps the file and hands out tensors one
by one, so a checkpoint is never held twice in host memory.

Counterpart in giveen/spite: the GGUF reader with typed errors for bad magic,
truncation and out-of-bounds offsets (crates/spite-loader/src/lib.rs:18-40,68-111).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

_TORCH = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
          "I8": torch.int8, "U8": torch.uint8, "I16": torch.int16, "I32": torch.int32,
          "I64": torch.int64, "BOOL": torch.bool}
_NAME = {v: k for k, v in _TORCH.items()}
_SIZE = {k: torch.empty(0, dtype=v).element_size() for k, v in _TORCH.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped file.  `entries[name] = (dtype string, shape tuple, begin, end)`."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: {size} bytes is too short for a safetensors header")
        self._fh = open(self.path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8 or hlen > 1 << 31:
            raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from None
        self._base = 8 + hlen
        self.metadata = header.pop("__metadata__", {})
        self.entries = {}
        for name, info in header.items():
            try:
                dt, shape = info["dtype"], tuple(int(x) for x in info["shape"])
                lo, hi = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: malformed header entry for {name!r}") from None
            if dt not in _TORCH:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dt}")
            n = 1
            for s in shape:
                n *= s
            if hi - lo != n * _SIZE[dt]:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} of shape {shape} and dtype {dt} needs "
                    f"{n * _SIZE[dt]} bytes, header gives {hi - lo}")
            if lo < 0 or self._base + hi > size:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} ends at byte {self._base + hi}, file has {size} (truncated?)")
            self.entries[name] = (dt, shape, lo, hi)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return list(self.entries)

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that owns its memory (copied out of the mapping)."""
        dt, shape, lo, hi = self.entries[name]
        if hi == lo:
            return torch.empty(shape, dtype=_TORCH[dt])
        buf = bytearray(self._map[self._base + lo:self._base + hi])
        return torch.frombuffer(buf, dtype=_TORCH[dt]).reshape(shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def save_file(tensors: dict[str, torch.Tensor], path, metadata: dict | None = None):
    """Write `tensors` (CPU, any of the supported dtypes) to one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = list(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAME:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAME[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            fh.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def open_checkpoint(folder) -> list[SafetensorsFile]:
    """The files of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` lists."""
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        try:
            names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        except (json.JSONDecodeError, KeyError) as e:
            raise SafetensorsError(f"{index}: cannot read weight_map ({e})") from None
        return [SafetensorsFile(folder / n) for n in names]
    single = folder / "model.safetensors"
    if not single.is_file():
        raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
    return [SafetensorsFile(single)]
