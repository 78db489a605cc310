"""What every architecture's configuration has to say, whatever its keys are.

An architecture's typed configuration (for instance `Qwen3Config`) reads its
own config.json keys and turns them into a `ModelPlan`: a description of the
layers as parts (mixer, feed-forward, norm, position encoding), layer by
layer, and the order in which they run.  The engine builds the model from the
plan alone; nothing below the plan knows which architecture it serves.

Upstream has one struct of ints per architecture and a model class that
hard-wires the layer (src/models/qwen3/qwen3.h:10-24, qwen3.cpp:205-253).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


class ConfigError(ValueError):
    """A config.json that cannot be served: a missing key, a wrong type, or an
    option this library does not compute."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: `kind` names a registered part class, `params` are
    its sizes and constants, `weights` maps the part's own tensor names to the
    names in the checkpoint."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    weights: dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A block: which arrangement, and the parts it arranges."""
    block: str                      # registered block arrangement, e.g. "pre_norm_residual"
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict[str, PartSpec]      # arrangement-specific names, e.g. {"input": ..., "post_mixer": ...}
    position: Optional[str] = None  # key into ModelPlan.positions, None = the mixer takes no positions


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer within a step.

    `layer` indexes ModelPlan.layers (the same layer may be named by several
    entries: its weights are then shared).  `cache` names the cache entry this
    run reads; `writes_cache` False means it only reads what another entry
    with the same `cache` wrote earlier in the step."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    positions: dict[str, PartSpec]
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def n_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)


def require(cfg: dict, key: str, typ, where: str = "config.json"):
    """cfg[key] as `typ`, or a ConfigError that names the key."""
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"{where}: key '{key}' is required")
    return coerce(cfg[key], key, typ, where)


def optional(cfg: dict, key: str, typ, default, where: str = "config.json"):
    if key not in cfg or cfg[key] is None:
        return default
    return coerce(cfg[key], key, typ, where)


def coerce(value, key: str, typ, where: str):
    if typ is int:
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value == int(value):
                return int(value)
            raise ConfigError(f"{where}: key '{key}' must be an integer, found {value!r}")
        return value
    if typ is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{where}: key '{key}' must be a number, found {value!r}")
        return float(value)
    if typ is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"{where}: key '{key}' must be true or false, found {value!r}")
        return value
    if typ is str:
        if not isinstance(value, str):
            raise ConfigError(f"{where}: key '{key}' must be a string, found {value!r}")
        return value
    if typ is list:
        if not isinstance(value, list):
            raise ConfigError(f"{where}: key '{key}' must be a list, found {value!r}")
        return value
    raise TypeError(typ)
