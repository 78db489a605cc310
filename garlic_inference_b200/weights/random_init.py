"""Random weights: a model folder (config.json, model.safetensors) from a
configuration and a seed, or tensors made directly on the device.

Matrices and tables are N(0, std); norm weights are norm_mean + N(0, norm_std).
Each tensor has a generator of its own, seeded by (seed, tensor name), so the
values do not depend on the order in which tensors are made.  Upstream has no
random-weights mode.
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path

import torch

from .loader import TensorWant
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1)


def random_tensor(name: str, want: TensorWant, seed: int, std: float, norm_mean: float, norm_std: float,
                  dtype: torch.dtype, device="cpu") -> torch.Tensor:
    device = torch.device(device)
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if want.role == "norm":
        t = torch.full(tuple(want.shape), float(norm_mean), dtype=torch.float32, device=device)
        if norm_std:
            t += torch.randn(tuple(want.shape), generator=g, dtype=torch.float32, device=device) * norm_std
        return t.to(dtype)
    if device.type == "cuda" and dtype == torch.bfloat16:
        # big matrices: draw in bfloat16 directly, no float32 copy of the whole tensor
        return torch.randn(tuple(want.shape), generator=g, dtype=dtype, device=device).mul_(std)
    return (torch.randn(tuple(want.shape), generator=g, dtype=torch.float32, device=device) * std).to(dtype)


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
                       norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write config.json and model.safetensors for `config` (an architecture's typed configuration)."""
    from ..engine.model import wanted_tensors
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    wants = wanted_tensors(config.plan())
    tensors = {name: random_tensor(name, want, seed, std, norm_mean, norm_std, dtype)
               for name, want in wants.items()}
    (model_dir / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    write_safetensors(model_dir / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": seed, "std": std, "norm_std": norm_std})
    return model_dir
