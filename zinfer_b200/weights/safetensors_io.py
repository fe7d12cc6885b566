"""Reader and writer of the safetensors container, used instead of the reference's GGUF reader
(src/gguf.zig:140-255): an 8-byte little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes.

The reader maps the file and checks every bound before it hands out a tensor, as the
reference's cursor does (src/gguf.zig:163-255): a truncated or inconsistent file gives a
`WeightFileError`, never a crash.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch


class WeightFileError(ValueError):
    """The container itself is malformed (not: a tensor the model wants is missing)."""


# safetensors dtype name -> (torch dtype, bytes per element)
_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int          # absolute offsets into the file
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file: `infos` by name, `tensor(name)` as a CPU tensor."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._f = open(self.path, "rb")
        except OSError as e:
            raise WeightFileError(f"{self.path}: cannot open ({e.strerror})") from e
        size = self.path.stat().st_size
        if size < 8:
            raise WeightFileError(f"{self.path}: {size} bytes is too short for a safetensors header")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > MAX_HEADER or 8 + hlen > size:
            raise WeightFileError(f"{self.path}: header length {hlen} does not fit the file of {size} bytes")
        try:
            header = json.loads(bytes(self._mm[8:8 + hlen]).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{self.path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise WeightFileError(f"{self.path}: header must be a JSON object")
        base = 8 + hlen
        self.metadata = header.pop("__metadata__", None) or {}
        self.infos: dict[str, TensorInfo] = {}
        for name, info in header.items():
            try:
                dt, shape, (a, b) = info["dtype"], info["shape"], info["data_offsets"]
                shape = tuple(int(s) for s in shape)
                a, b = int(a), int(b)
            except (KeyError, TypeError, ValueError) as e:
                raise WeightFileError(f"{self.path}: tensor '{name}' has a malformed entry ({e})") from e
            if dt not in _DTYPES:
                raise WeightFileError(f"{self.path}: tensor '{name}' has unsupported dtype {dt}")
            tdt, esz = _DTYPES[dt]
            if any(s < 0 for s in shape):
                raise WeightFileError(f"{self.path}: tensor '{name}' has a negative dimension {shape}")
            count = 1
            for s in shape:
                count *= s
            if a < 0 or b < a or base + b > size:
                raise WeightFileError(f"{self.path}: tensor '{name}' data [{a}, {b}) lies outside the file")
            if b - a != count * esz:
                raise WeightFileError(
                    f"{self.path}: tensor '{name}' of shape {shape} and dtype {dt} needs {count * esz} bytes, has {b - a}")
            self.infos[name] = TensorInfo(name, tdt, shape, base + a, base + b)

    def __contains__(self, name: str) -> bool:
        return name in self.infos

    def names(self) -> list[str]:
        return list(self.infos)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns a copy of the named tensor's data."""
        info = self.infos[name]
        n = info.end - info.begin
        if n == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=n, offset=info.begin).copy()
        return torch.from_numpy(raw).view(info.dtype).reshape(info.shape)

    def close(self) -> None:
        try:
            self._mm.close()
        finally:
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Writes CPU tensors in the order given, data back to back as the format requires."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightFileError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        data = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(data)]}
        blobs.append(data)
        offset += len(data)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((-len(hjson)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for b in blobs:
            f.write(b)
