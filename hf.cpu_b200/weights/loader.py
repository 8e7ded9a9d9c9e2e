"""Weights by tensor name, with one error that lists everything wrong at once.

A model declares the tensors it needs as :class:`TensorSpec` (name, shape, how
to initialise it at random).  ``load_tensors`` reads exactly those from a model
folder's ``model.safetensors`` and reports missing tensors, unexpected tensors
and wrong shapes in a single :class:`WeightError`.

Dtype policy: floating tensors are kept in the run dtype's storage type — for a
bfloat16 run, 16-bit tensors become bfloat16 and a tensor stored in 32-bit stays
32-bit; for a float32 run everything floating is widened to float32 (exact for
bf16/f16).  Integer tensors become int32.

The reference checks each tensor's shape against the hyper-parameters and names
the tensor and both shapes in its message (src/model.c:60-61, :79-82).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

from .safetensors_io import SafetensorsFile, WeightFormatError


class WeightError(ValueError):
    """Tensors are missing, unexpected or misshapen; the message lists all of them."""

    def __init__(self, path, missing, unexpected, misshapen, other=()):
        self.missing, self.unexpected, self.misshapen = list(missing), list(unexpected), list(misshapen)
        lines = [f"{path}: the weights do not match the configuration"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.misshapen:
            lines.append(f"  tensor '{name}' has shape {'x'.join(map(str, got)) or 'scalar'}, "
                         f"expected {'x'.join(map(str, want)) or 'scalar'}")
        lines += [f"  {o}" for o in other]
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"        # "normal": N(0, std); "norm": 1 + N(0, std/2); "int": small integers
    optional: bool = False


def storage_dtype(stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def weights_path(folder: str) -> str:
    return os.path.join(folder, "model.safetensors")


def load_tensors(folder: str, specs: Iterable[TensorSpec], run_dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    path = weights_path(folder)
    specs = list(specs)
    want = {s.name: s for s in specs}
    try:
        f = SafetensorsFile(path)
    except WeightFormatError:
        raise
    with f:
        have = set(f.names())
        missing = [s.name for s in specs if s.name not in have and not s.optional]
        unexpected = sorted(have - set(want))
        misshapen = [(n, f.shape(n), tuple(want[n].shape)) for n in sorted(have & set(want))
                     if tuple(f.shape(n)) != tuple(want[n].shape)]
        other = [f"tensor '{n}' has dtype {f.dtype(n)}, which is neither floating nor integer"
                 for n in sorted(have & set(want)) if f.dtype(n) == torch.bool]
        if missing or unexpected or misshapen or other:
            raise WeightError(path, missing, unexpected, misshapen, other)
        out = {}
        for s in specs:
            if s.name not in have:
                continue
            t = f.tensor(s.name)
            out[s.name] = t.to(storage_dtype(t.dtype, run_dtype)).to(device)
        return out
