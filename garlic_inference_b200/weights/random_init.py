"""Random weights: a model folder (config.json, model.safetensors) from a
configuration and a seed, or tensors made directly on the device.

Matrices and tables are N(0, std); norm weights are norm_mean + N(0, norm_std).
The generator is counter-based: element i of a tensor depends on (seed, tensor
name, i) and nothing else, so the values do not depend on the order in which
tensors are made, nor on where: `normal_values` below (numpy, on the host)
and the kernel `gi_random_normal` (csrc/random_init.cu, on the device) do the
same integer hashing and the same two float32 operations, and give the same
bits.  A folder written on the CPU and a model initialised on the GPU from the
same seed are therefore the same model.  Upstream has no random-weights mode.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from .loader import TensorWant
from .safetensors_io import write_safetensors_lazy

_MASK = (1 << 64) - 1
_CHUNK = 1 << 22                 # elements hashed at a time on the host


def _mix64_int(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's random stream: the seed hashed with the FNV-1a hash of its name."""
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return _mix64_int(_mix64_int(int(seed) & _MASK) ^ h)


def normal_values(key: int, n: int, mean: float, std: float, start: int = 0) -> np.ndarray:
    """float32 values mean + std * z_i for i in [start, start + n): z_i is the centred sum of twelve 16-bit
    fields of three hashes of (key, i), scaled by 2^-16 (variance 1 - 2^-32, cut at +-6)."""
    out = np.empty(n, dtype=np.float32)
    k, m16 = np.uint64(key), np.uint64(0xFFFF)
    mean32, std32 = np.float32(mean), np.float32(std)
    with np.errstate(over="ignore"):
        for c0 in range(0, n, _CHUNK):
            i3 = np.arange(start + c0, start + min(n, c0 + _CHUNK), dtype=np.uint64) * np.uint64(3)
            s = np.zeros(i3.size, dtype=np.int64)
            for j in range(3):
                h = _mix64(k ^ (i3 + np.uint64(j)))
                s += ((h & m16) + ((h >> np.uint64(16)) & m16) + ((h >> np.uint64(32)) & m16)
                      + (h >> np.uint64(48))).astype(np.int64)
            z = (2 * s - 786420).astype(np.float32) * np.float32(2.0 ** -17)
            out[c0:c0 + i3.size] = mean32 + std32 * z            # two float32 roundings, as on the device
    return out


def random_tensor(name: str, want: TensorWant, seed: int, std: float, norm_mean: float, norm_std: float,
                  dtype: torch.dtype, device="cpu") -> torch.Tensor:
    device = torch.device(device)
    mean, dev = (norm_mean, norm_std) if want.role == "norm" else (0.0, std)
    key = tensor_key(seed, name)
    if device.type == "cuda":
        from ..ops import kernels
        with torch.cuda.device(device):
            return kernels.random_normal(torch.empty(tuple(want.shape), dtype=dtype, device=device), key, mean, dev)
    n = 1
    for d in want.shape:
        n *= int(d)
    return torch.from_numpy(normal_values(key, n, mean, dev)).reshape(tuple(want.shape)).to(dtype)


class RandomSource:
    """Tensor source that makes each tensor when it is asked for (nothing touches the disk)."""

    def __init__(self, wants: dict[str, TensorWant], seed: int = 0, std: float = 0.02, norm_mean: float = 1.0,
                 norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16, device="cpu"):
        self.wants, self.seed, self.std = wants, seed, std
        self.norm_mean, self.norm_std, self.dtype, self.device = norm_mean, norm_std, dtype, device

    def stored_dtype(self, name: str) -> torch.dtype:
        return self.dtype

    def tensor(self, name: str) -> torch.Tensor:
        return random_tensor(name, self.wants[name], self.seed, self.std, self.norm_mean, self.norm_std,
                             self.dtype, self.device)


def write_random_model(model_dir, config, seed: int = 0, std: float = 0.02, norm_mean: float = 1.0,
                       norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16, device="cpu") -> Path:
    """Write config.json and model.safetensors for `config` (an architecture's typed configuration).  With a
    CUDA `device` the values are made there and copied back (the same values, much faster for large models)."""
    from ..engine.model import wanted_tensors
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    wants = wanted_tensors(config.plan())

    (model_dir / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    write_safetensors_lazy(
        model_dir / "model.safetensors", {name: (dtype, tuple(want.shape)) for name, want in wants.items()},
        lambda name: random_tensor(name, wants[name], seed, std, norm_mean, norm_std, dtype, device),
        metadata={"format": "pt", "seed": seed, "std": std, "norm_std": norm_std})
    return model_dir
