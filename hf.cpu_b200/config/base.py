"""Typed configuration: the base class, the plan a configuration expands to, and errors.

A configuration is read from the architecture's own ``config.json`` keys and is
the only source of sizes and constants; nothing downstream hard-codes one.  A
configuration expands to a :class:`ModelPlan`, which is plain data: the parts of
each layer (kind + arguments), and the order in which layers run.

The reference keeps the same information in ``hfc_hparams`` (src/model.h:23-29)
and fills it from GGUF metadata with defaults and plausibility checks
(src/model.c:119-145).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, ClassVar, Dict, List, Optional


class ConfigError(ValueError):
    """A configuration key is missing, mistyped or out of range."""


class UnsupportedError(ConfigError):
    """The configuration asks for something this engine does not implement."""


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name from a registry, with all of its constants as arguments."""
    kind: str
    args: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer with weights of its own: a block arrangement over four parts.

    ``prefix`` is the checkpoint name prefix of the layer's tensors.
    """
    prefix: str
    block: PartSpec
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.

    ``layer`` indexes ``ModelPlan.layers`` (a layer may appear more than once).
    ``cache_of`` names an *earlier entry* whose cache this entry's mixer reads
    instead of keeping one of its own; ``None`` means the entry owns its cache.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    positions: Dict[str, PartSpec]          # shared position encodings, by name
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: List[int] = field(default_factory=list)

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, plan has {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                                      f"which is not an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                                      f"which has none of its own")


@dataclass
class ModelConfig:
    """Base of every architecture's configuration."""

    # the name the registry resolved (``architectures[0]`` or ``model_type``)
    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        arch = d.pop("architecture", "")
        d["architectures"] = [arch]
        return d

    def plan(self) -> ModelPlan:
        raise NotImplementedError

    # ---- the GGUF side of an architecture (optional) ------------------------------------------------------
    # ``general.architecture`` of the files this class reads and writes; the class is registered under it
    gguf_architecture: ClassVar[Optional[str]] = None

    @classmethod
    def from_gguf(cls, meta: Dict[str, Any], shapes: Dict[str, tuple], where: str = "") -> "ModelConfig":
        """The configuration a GGUF file's metadata describe.  ``shapes`` gives the shape (rows first) of every
        tensor by its name in the file, for what the metadata leave to the tensors (the vocabulary size)."""
        raise UnsupportedError(f"architecture '{cls.__name__}' does not read GGUF metadata")

    def gguf_metadata(self) -> List[tuple]:
        """(key, value type, value) for every metadata key of this configuration, with the format's type ids
        (4 = u32, 6 = f32, 8 = string)."""
        raise UnsupportedError(f"architecture '{type(self).__name__}' does not write GGUF metadata")

    def gguf_names(self) -> Dict[str, str]:
        """Checkpoint tensor name -> name in a GGUF file, for every tensor such a file stores."""
        raise UnsupportedError(f"architecture '{type(self).__name__}' has no GGUF tensor names")

    def gguf_left_out(self) -> List[str]:
        """Checkpoint tensors that an export leaves out on purpose (a tied head's copy of the embedding)."""
        return []

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=1, sort_keys=True)


# ---- helpers to read typed keys -------------------------------------------------------------

_MISSING = object()


def take_int(d: Dict[str, Any], key: str, default: Any = _MISSING, lo: int = None, hi: int = None) -> int:
    v = d.get(key, _MISSING)
    if v is _MISSING or v is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    if isinstance(v, bool) or not isinstance(v, int):
        if isinstance(v, float) and v == int(v):
            v = int(v)
        else:
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if lo is not None and v < lo or hi is not None and v > hi:
        raise ConfigError(f"config.json: '{key}' = {v} is outside [{lo}, {hi}]")
    return v


def take_float(d: Dict[str, Any], key: str, default: Any = _MISSING, lo: float = None) -> float:
    v = d.get(key, _MISSING)
    if v is _MISSING or v is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    v = float(v)
    if lo is not None and not v > lo:
        raise ConfigError(f"config.json: '{key}' = {v} must be greater than {lo}")
    return v


def take_bool(d: Dict[str, Any], key: str, default: bool) -> bool:
    v = d.get(key, None)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
    return v
