"""One registry from the architecture's name (config.json `model_type`) to its parser and its model.

The reference keeps a map from model_type to architecture and fails with the list of
supported names (src/main/java/org/robomiri/jllm/model/Families.java:28-50,100-105).
Here an entry holds two callables: `parse(config_dict) -> spec` and
`build(spec, tensors, runtime) -> model`; the second defaults to the generic decoder
built from parts.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Optional

from .specs import ConfigError


@dataclass(frozen=True)
class ArchitectureEntry:
    model_type: str
    parse: Callable[[dict], object]
    build: Optional[Callable] = None       # None = the generic decoder of engine.model


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(model_type: str, parse: Callable[[dict], object], build: Optional[Callable] = None,
                          replace: bool = False) -> None:
    if model_type in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {model_type!r} is registered already")
    _ARCHITECTURES[model_type] = ArchitectureEntry(model_type, parse, build)


def unregister_architecture(model_type: str) -> None:
    _ARCHITECTURES.pop(model_type, None)


def supported_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_entry(model_type: str) -> ArchitectureEntry:
    if model_type not in _ARCHITECTURES:
        raise ConfigError(f"unsupported model_type {model_type!r} (supported: {', '.join(supported_architectures())})")
    return _ARCHITECTURES[model_type]


def parse_config(values: dict):
    """config.json as a dict -> the typed spec of its architecture."""
    if not isinstance(values, dict):
        raise ConfigError("config.json must hold a JSON object")
    model_type = values.get("model_type")
    if not isinstance(model_type, str):
        raise ConfigError("config.json: required key 'model_type' is missing")
    return architecture_entry(model_type).parse(values)


def load_config(model_dir) -> tuple:
    """(spec, raw dict) of `model_dir/config.json`."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        values = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    return parse_config(values), values
