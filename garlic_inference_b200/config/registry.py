"""The one registry from an architecture's name to its model.

config.json's `architectures[0]` picks the entry by exact match; an unknown
name is an error that lists the known ones.  Upstream matches by substring in
an if-chain and falls off the end of the function for an unknown name
(src/models/model.cpp:10-34).

An entry is the architecture's typed configuration class.  That class reads
the architecture's own keys (`from_dict`), writes them back (`to_dict`) and
describes the model as parts (`plan() -> ModelPlan`); the engine builds the
model from the plan.
"""
from __future__ import annotations

import json
from pathlib import Path

from .base import ConfigError

_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    for attr in ("from_dict", "to_dict", "plan"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"configuration class for {name!r} lacks {attr}()")
    _ARCHITECTURES[name] = config_cls


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; registered: "
                          f"{', '.join(known_architectures()) or '(none)'}") from None


def load_config(model_dir):
    """Typed configuration of the model folder, chosen by `architectures[0]`."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and "
                          "model.safetensors)")
    try:
        cfg = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from None
    archs = cfg.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{path}: key 'architectures' must be a non-empty list of names")
    return config_class_for(archs[0]).from_dict(cfg, str(path))
