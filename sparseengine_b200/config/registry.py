"""One registry from an architecture's name to the code that builds its model.

The reference keeps ``MODEL_SPECS[model_type].runtime_class_name`` and looks the class
up in the model runner's globals (src/sparseengine/models/spec.py:103-211,
src/sparseengine/engine/model_runner.py:150-161).  Here an architecture registers a
typed configuration class (read from its own ``config.json`` keys) and a builder that
returns a :class:`~sparseengine_b200.config.specs.ModelSpec`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable

from .specs import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(dict) -> typed config
    build: Callable[[Any], ModelSpec]      # typed config -> ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build: Callable[[Any], ModelSpec]) -> None:
    """Register (or replace) an architecture under the name ``config.json`` gives in
    ``architectures[0]``."""
    _ARCHITECTURES[name] = Architecture(name, config_class, build)


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(config: dict) -> Architecture:
    names = config.get("architectures") or []
    if not isinstance(names, (list, tuple)) or len(names) != 1:
        raise ValueError(f"config.json must name exactly one architecture, got {names!r}")
    name = names[0]
    if name not in _ARCHITECTURES:
        raise ValueError(
            f"unknown architecture {name!r}; registered: {architectures()}")
    return _ARCHITECTURES[name]


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir!r}")
    with open(path) as f:
        return json.load(f)


def load_model_spec(model_dir_or_dict) -> tuple[Any, ModelSpec]:
    """Return ``(typed config, ModelSpec)`` for a model folder or a config dictionary."""
    raw = model_dir_or_dict if isinstance(model_dir_or_dict, dict) else read_config_json(model_dir_or_dict)
    arch = resolve_architecture(raw)
    typed = arch.config_class.from_dict(raw)
    return typed, arch.build(typed)
