"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

FeLLM's built-in path has no such table (crates/fellm-model/src/lib.rs:3-4 infers topology from
tensor names); its plugin host keeps one (crates/fellm-plugin-host/src/registry.rs:44) and the
DSpark plugin checks `architectures[0]` against a list (plugins/dspark/src/lib.rs:66-76).

An architecture is two functions: `read_config(dict) -> typed config` and
`build_spec(config) -> ModelSpec` (fellm_b200.parts.spec).  Everything below the spec - parts,
cache, step function, kernels - never learns the architecture's name.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict

from .errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable        # dict -> typed config
    build_spec: Callable         # typed config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, read_config: Callable, build_spec: Callable) -> Architecture:
    arch = Architecture(name, read_config, build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def architectures():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES))}")
    return _ARCHITECTURES[name]


def read_model_config(folder):
    """(architecture, typed config) of the model folder's config.json."""
    path = Path(folder) / "config.json"
    try:
        d = json.loads(path.read_text())
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {folder}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)


def config_from_dict(d: dict):
    archs = d.get("architectures") or []
    if not archs:
        raise ConfigError("config.json: missing key 'architectures'")
    arch = get_architecture(str(archs[0]))
    return arch, arch.read_config(d)


def _load_builtin():
    # importing the module registers it
    from ..models import lfm2  # noqa: F401
