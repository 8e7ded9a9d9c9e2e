"""Random weights from a configuration and a seed.

Matrices and biases are N(0, std), norm weights 1 + N(0, std/2).  Each tensor
has its own generator keyed by the seed and the tensor's name, so the values do
not depend on the order of creation.  The reference's generator for its tests is
tools/mkmodel.pl (seeded, per-tensor scales, tools/mkmodel.pl:104-119).
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict, Iterable

import torch

from .loader import TensorSource, TensorSpec, weights_path
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def _draw(s: TensorSpec, seed: int, dtype: torch.dtype, device: torch.device, std: float) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, s.name))
    if s.init == "int":
        return torch.randint(0, 8, s.shape, generator=g, device=device, dtype=torch.int32)
    # drawn in float32 on the target device
    t = torch.empty(s.shape, dtype=torch.float32, device=device).normal_(0.0, 1.0, generator=g)
    t = 1.0 + t * (std / 2) if s.init == "norm" else t * std
    return t.to(dtype)


def random_tensors(specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype,
                   device: torch.device = torch.device("cpu"), std: float = 0.02) -> Dict[str, torch.Tensor]:
    device = torch.device(device)
    return {s.name: _draw(s, seed, dtype, device, std) for s in specs}


class RandomSource(TensorSource):
    """Random tensors made when they are asked for, one at a time, with the values of :func:`random_tensors`."""

    def __init__(self, specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype, device: torch.device,
                 std: float = 0.02):
        super().__init__(dtype, device)
        self.specs = {s.name: s for s in specs}
        self.seed, self.dtype, self.std = seed, dtype, std

    def names(self):
        return self.specs.keys()

    def __contains__(self, name):
        return name in self.specs

    def meta(self, name):
        s = self.specs[name]
        return (torch.int32 if s.init == "int" else self.dtype), tuple(s.shape)

    def _make(self, name):
        return _draw(self.specs[name], self.seed, self.dtype, self.device, self.std)


def write_random_model(config, folder: str, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a ModelConfig) into ``folder``."""
    from ..models import build_model_specs
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    source = RandomSource(build_model_specs(config), seed, dtype, torch.device("cpu"), std=std)
    write_safetensors(weights_path(folder), source, metadata={"format": "pt"})
    return folder
