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

from .loader import TensorSpec, weights_path
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensors(specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype,
                   device: torch.device = torch.device("cpu"), std: float = 0.02) -> Dict[str, torch.Tensor]:
    out = {}
    device = torch.device(device)
    for s in specs:
        g = torch.Generator(device=device)
        g.manual_seed(_seed_for(seed, s.name))
        if s.init == "int":
            out[s.name] = torch.randint(0, 8, s.shape, generator=g, device=device, dtype=torch.int32)
            continue
        # draw in float32 on the target device, one tensor at a time
        t = torch.empty(s.shape, dtype=torch.float32, device=device).normal_(0.0, 1.0, generator=g)
        if s.init == "norm":
            t = 1.0 + t * (std / 2)
        else:
            t = t * std
        out[s.name] = t.to(dtype)
    return out


def write_random_model(config, folder: str, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a ModelConfig) into ``folder``."""
    from ..models import build_model_specs
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    tensors = random_tensors(build_model_specs(config), seed, dtype, std=std)
    write_safetensors(weights_path(folder), tensors, metadata={"format": "pt"})
    return folder
