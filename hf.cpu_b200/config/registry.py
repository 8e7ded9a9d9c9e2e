"""One registry from an architecture's name to its configuration class.

The reference gates on ``general.architecture`` with string compares and answers
anything else with "architecture '%s' is not supported yet" (src/model.c:107-110).
Here the names are ``config.json``'s ``architectures[0]`` and ``model_type``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Type

from .base import ConfigError, ModelConfig, UnsupportedError

_ARCHITECTURES: Dict[str, Type[ModelConfig]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig]) -> None:
    """Make ``name`` (as found in config.json) resolve to ``config_cls``."""
    _ARCHITECTURES[name] = config_cls


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(d: Dict[str, Any]) -> str:
    names = []
    archs = d.get("architectures")
    if isinstance(archs, list):
        names += [a for a in archs if isinstance(a, str)]
    if isinstance(d.get("model_type"), str):
        names.append(d["model_type"])
    if not names:
        raise ConfigError("config.json: neither 'architectures' nor 'model_type' names an architecture")
    for n in names:
        if n in _ARCHITECTURES:
            return n
    raise UnsupportedError(f"architecture '{names[0]}' is not supported yet "
                           f"(known: {', '.join(known_architectures())})")


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    name = resolve_architecture(d)
    cfg = _ARCHITECTURES[name].from_dict(d)
    cfg.architecture = name
    return cfg


def config_from_gguf(meta: Dict[str, Any], shapes: Dict[str, tuple], where: str = "") -> ModelConfig:
    """The configuration of a GGUF file, through the class registered under its ``general.architecture``."""
    arch = meta.get("general.architecture")
    if not isinstance(arch, str):
        raise ConfigError(f"{where}: general.architecture is missing")
    cls = _ARCHITECTURES.get(arch)
    known = sorted(n for n, c in _ARCHITECTURES.items() if getattr(c, "gguf_architecture", None) == n)
    if arch not in known:
        raise UnsupportedError(f"architecture '{arch}' is not supported yet (known: {', '.join(known)})")
    cfg = cls.from_gguf(meta, shapes, where)
    cfg.architecture = arch
    return cfg


def load_config(folder: str) -> ModelConfig:
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)
