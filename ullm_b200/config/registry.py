"""The one registry from an architecture's name (config.json "architectures")
to what builds its model: a parser of its config.json keys and a translation of
that typed config into a ModelSpec.  ullm/models/registry.py:3-5 and the lookup
in ullm/core/model_runner.py:186-194 are the counterparts.

Adding an architecture = one `register_architecture` call; nothing else in the
framework names an architecture.
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
    parse_config: Callable[[dict[str, Any]], Any]  # config.json dict -> typed config
    model_spec: Callable[[Any], ModelSpec]  # typed config -> ModelSpec


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, model_spec) -> Architecture:
    arch = Architecture(name, parse_config, model_spec)
    ARCHITECTURES[name] = arch
    return arch


def resolve_architecture(config: dict[str, Any]) -> Architecture:
    names = config.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in ARCHITECTURES:
            return ARCHITECTURES[n]
    raise ValueError(
        f"Model arch {names} not supported. Registered architectures: {sorted(ARCHITECTURES)}"
    )


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and *.safetensors")
    with open(path) as f:
        return json.load(f)


def load_model_spec(model_dir_or_dict) -> tuple[Any, ModelSpec]:
    """(typed config, ModelSpec) for a model folder or a config.json dict."""
    d = model_dir_or_dict if isinstance(model_dir_or_dict, dict) else read_config_json(model_dir_or_dict)
    arch = resolve_architecture(d)
    cfg = arch.parse_config(d)
    spec = arch.model_spec(cfg)
    spec.validate()
    return cfg, spec
