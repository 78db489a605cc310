"""Weights of a model folder, by tensor name.

A folder holds either `model.safetensors` or shards named by
`model.safetensors.index.json["weight_map"]` (upstream: src/models/loader.h:212-231).
Before anything is copied to the GPU the whole list of tensors the model
wants is compared with what the folder has, and ONE error lists everything
that is wrong: missing tensors, wrong shapes, wrong types, with the tensors
the model does not use listed beside them.  Tensors the model does not use
are no error by themselves (a tied model whose file still stores
`lm_head.weight`, a stray buffer): they are listed once in a
`SurplusTensorWarning` and left on the disk, as upstream leaves them
(src/models/qwen3/qwen3.cpp:58 never reads a stored head).  Upstream checks no
shape and reports a missing tensor only when it is first read
(loader.h:60-62, 234, 249).

Precision on the device (`device_dtype`): a tensor stored in bfloat16 or
float16 is kept in bfloat16, a tensor stored in 32-bit floating point stays
32-bit, integer tables become int32; under the float32 engine every floating
tensor is widened to float32 (exactly).
"""
from __future__ import annotations

import json
import warnings
from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The folder's tensors do not fit the model; the message lists every mismatch."""


class SurplusTensorWarning(UserWarning):
    """The folder holds tensors that the model does not use; the message lists them."""


@dataclass(frozen=True)
class TensorWant:
    shape: tuple
    role: str = "matrix"        # "matrix" | "norm" | "table": used by random initialisation


class Checkpoint:
    """All tensors of a model folder, whichever file holds them."""

    def __init__(self, model_dir):
        self.model_dir = Path(model_dir)
        index = self.model_dir / "model.safetensors.index.json"
        single = self.model_dir / "model.safetensors"
        self._files: dict[str, SafetensorsFile] = {}
        self._where: dict[str, str] = {}
        try:
            if index.is_file():
                weight_map = json.loads(index.read_text()).get("weight_map")
                if not isinstance(weight_map, dict):
                    raise WeightError(f"{index}: no 'weight_map' object")
                for shard in sorted(set(weight_map.values())):
                    self._files[shard] = SafetensorsFile(self.model_dir / shard)
                for name, shard in weight_map.items():
                    if name not in self._files[shard].names():
                        raise WeightError(f"{index}: '{name}' is mapped to {shard}, which does not hold it")
                    self._where[name] = shard
            elif single.is_file():
                self._files[single.name] = SafetensorsFile(single)
                for name in self._files[single.name].names():
                    self._where[name] = single.name
            else:
                raise WeightError(f"{self.model_dir}: neither model.safetensors nor "
                                  "model.safetensors.index.json")
        except SafetensorsError as e:
            raise WeightError(str(e)) from None

    def names(self) -> list[str]:
        return list(self._where)

    def shape(self, name: str) -> tuple:
        return self._files[self._where[name]].info(name)["shape"]

    def stored_dtype(self, name: str) -> torch.dtype:
        from .safetensors_io import DTYPES
        return DTYPES[self._files[self._where[name]].info(name)["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def check(self, wanted: dict[str, TensorWant]) -> None:
        have = set(self._where)
        missing = [n for n in wanted if n not in have]
        unexpected = sorted(have - set(wanted))
        wrong = [(n, tuple(w.shape), self.shape(n)) for n, w in wanted.items()
                 if n in have and tuple(self.shape(n)) != tuple(w.shape)]
        not_float = [(n, self.stored_dtype(n)) for n, w in wanted.items()
                     if n in have and w.role != "index" and not self.stored_dtype(n).is_floating_point]
        self.unexpected = unexpected
        if not (missing or wrong or not_float):
            if unexpected:
                shown = ", ".join(f"{n} {list(self.shape(n))}" for n in unexpected[:20])
                more = f" and {len(unexpected) - 20} more" if len(unexpected) > 20 else ""
                warnings.warn(f"{self.model_dir}: {len(unexpected)} tensors are not used by the model and were "
                              f"not loaded: {shown}{more}", SurplusTensorWarning, stacklevel=2)
            return
        lines = [f"{self.model_dir}: the tensors do not fit the model "
                 f"({len(missing)} missing, {len(unexpected)} unexpected, {len(wrong)} of wrong shape)"]
        lines += [f"  missing:    {n}  {list(wanted[n].shape)}" for n in missing]
        lines += [f"  unexpected: {n}  {list(self.shape(n))}" for n in unexpected]
        lines += [f"  wrong shape: {n}  wanted {list(w)}, found {list(f)}" for n, w, f in wrong]
        lines += [f"  wrong dtype: {n}  wanted floating point, found {d}" for n, d in not_float]
        raise WeightError("\n".join(lines))


def device_dtype(stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    """Precision in which a stored tensor is kept on the device (see the module text)."""
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if engine_dtype == torch.bfloat16:
        return torch.float32 if stored == torch.float32 else torch.bfloat16
    raise ValueError(f"engine dtype must be bfloat16 or float32, not {engine_dtype}")
