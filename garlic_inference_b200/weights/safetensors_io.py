"""Reading and writing safetensors files without any helper package.

Format: an 8-byte little-endian header length, a JSON header that maps each
tensor name to {dtype, shape, data_offsets}, then the raw bytes
(upstream reads the same, src/models/loader.h:30-54, without checking offsets).
The reader maps the file and hands out tensors that view the mapping; it
checks that each tensor's bytes lie inside the file and match its shape.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import numpy as np
import torch

# name in the file -> (torch dtype, bytes per element)
DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped .safetensors file: `names()`, `info(name)`, `tensor(name)`."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path}: no such file")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: shorter than its 8-byte header length")
        self._fh = open(self.path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} runs past the end of the "
                                   f"file ({size} bytes): truncated or not a safetensors file")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from None
        self._base = 8 + hlen
        self._entries: dict[str, dict] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dtype = info.get("dtype")
            if dtype not in DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has dtype {dtype!r}; "
                                       f"readable: {', '.join(DTYPES)}")
            shape = tuple(int(s) for s in info["shape"])
            lo, hi = (int(o) for o in info["data_offsets"])
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if hi - lo != numel * DTYPES[dtype][1]:
                raise SafetensorsError(f"{self.path}: tensor '{name}' of shape {list(shape)} {dtype} "
                                       f"needs {numel * DTYPES[dtype][1]} bytes, its offsets give {hi - lo}")
            if lo < 0 or self._base + hi > size:
                raise SafetensorsError(f"{self.path}: tensor '{name}' ends at byte {self._base + hi}, "
                                       f"the file has {size}: truncated")
            self._entries[name] = {"dtype": dtype, "shape": shape, "lo": lo, "hi": hi}

    def names(self) -> list[str]:
        return list(self._entries)

    def info(self, name: str) -> dict:
        return self._entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only: copy before writing)."""
        e = self._entries[name]
        dtype = DTYPES[e["dtype"]][0]
        numel = int(np.prod(e["shape"], dtype=np.int64)) if e["shape"] else 1
        if numel == 0:
            return torch.empty(e["shape"], dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # "buffer is not writable": it is only read
            t = torch.frombuffer(self._map, dtype=dtype, count=numel, offset=self._base + e["lo"])
        return t.view(e["shape"])

    def close(self):
        # tensors handed out keep the mapping alive; closing is only for files never read
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass
        self._fh.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write `tensors` (CPU, any of the readable dtypes) to one file, in the given order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which cannot be written")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, t in tensors.items():
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)


def write_safetensors_lazy(path, entries: dict, make, metadata: dict | None = None) -> None:
    """The same file, with each tensor made when its turn to be written comes: `entries` maps a name to
    (dtype, shape), `make(name)` returns that tensor.  Only one tensor is in memory at a time."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, (dtype, shape) in entries.items():
        if dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {dtype}, which cannot be written")
        nbytes = int(np.prod(shape, dtype=np.int64)) * torch.empty(0, dtype=dtype).element_size() if len(shape) else \
            torch.empty(0, dtype=dtype).element_size()
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(d) for d in shape],
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, (dtype, shape) in entries.items():
            t = make(name).detach().contiguous().cpu()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"tensor '{name}' was announced as {dtype} {list(shape)} and made as "
                                       f"{t.dtype} {list(t.shape)}")
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
