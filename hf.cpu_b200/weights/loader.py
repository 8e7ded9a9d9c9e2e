"""Weights by tensor name, one tensor at a time, with one error that lists everything wrong at once.

A model declares the tensors it needs as :class:`TensorSpec` (name, shape, how to initialise it at
random).  ``load_tensors`` opens a model folder's safetensors files, checks the directory of every file
against the specs and reports missing tensors, unexpected tensors and wrong shapes in a single
:class:`WeightError`.  No tensor data has been read at that point: what comes back is a
:class:`TensorSource`, a read-only mapping that reads, converts and uploads a tensor when a part asks
for it, so that the device never holds more than the weights bound so far plus the one in transit.

A folder may hold ``model.safetensors``, or ``model.safetensors.index.json`` with the shards it names
(``model-00001-of-0000N.safetensors`` ...), or, without an index, any number of ``*.safetensors`` files.
A name found in two files, or an index that names a file that is not there, is a format error.

Dtype policy: floating tensors are kept in the run dtype's storage type: for a bfloat16 run, 16-bit
tensors become bfloat16 and a tensor stored in 32-bit stays 32-bit; for a float32 run everything
floating is widened to float32 (exact for bf16/f16).  Integer tensors become int32.

The reference maps its model file once, read-only, and never copies it (src/model.h:3, src/pal.c:33-52);
it checks each tensor's shape against the hyper-parameters in one pass and names the tensor and both
shapes in its message (src/model.c:60-61, :79-82, :95-191).
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .safetensors_io import SafetensorsFile, WeightFormatError

SINGLE_FILE = "model.safetensors"
INDEX_FILE = SINGLE_FILE + ".index.json"


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
    """Where a model written by this package keeps its one weights file."""
    return os.path.join(folder, SINGLE_FILE)


def find_weight_files(folder: str) -> Tuple[List[str], Optional[Dict[str, str]]]:
    """The safetensors files of a model folder and, when the folder has an index, its map from tensor name to
    file name.  Order of preference: the single file, the index and its shards, every ``*.safetensors``."""
    single = os.path.join(folder, SINGLE_FILE)
    if os.path.isfile(single):
        return [single], None
    index_path = os.path.join(folder, INDEX_FILE)
    if os.path.isfile(index_path):
        try:
            with open(index_path) as f:
                index = json.load(f)
            wmap = index["weight_map"]
            if not isinstance(wmap, dict) or not all(isinstance(k, str) and isinstance(v, str) for k, v in wmap.items()):
                raise TypeError
        except (ValueError, KeyError, TypeError):
            raise WeightFormatError(f"{index_path}: not an index (a JSON object with a 'weight_map' from tensor "
                                    f"names to file names)") from None
        files = sorted(set(wmap.values()))
        for name in files:
            if os.path.basename(name) != name or not name:
                raise WeightFormatError(f"{index_path}: file name '{name}' leaves the model folder")
        absent = [n for n in files if not os.path.isfile(os.path.join(folder, n))]
        if absent:
            raise WeightFormatError(f"{index_path}: the index names {', '.join(absent)}, which "
                                    f"{'is' if len(absent) == 1 else 'are'} not in the folder")
        if not files:
            raise WeightFormatError(f"{index_path}: the index names no file")
        return [os.path.join(folder, n) for n in files], dict(wmap)
    files = sorted(glob.glob(os.path.join(glob.escape(folder), "*.safetensors")))
    if not files:
        if not os.path.isdir(folder):
            raise WeightFormatError(f"{folder}: no such folder")
        raise WeightFormatError(f"{single}: no such file (and the folder holds neither {INDEX_FILE} nor any "
                                f"other *.safetensors file)")
    return files, None


class TensorSource:
    """A read-only mapping from tensor name to tensor that makes a tensor when it is asked for.

    ``source[name]`` returns the tensor on the run's device in its storage dtype; every call makes a new one
    unless the name was marked with :meth:`keep` (a tensor that two parts bind, such as a tied head).
    ``meta(name)`` tells dtype and shape without touching data."""

    def __init__(self, run_dtype: torch.dtype, device: torch.device):
        self.run_dtype, self.device = run_dtype, torch.device(device)
        self._keep: set = set()
        self._kept: Dict[str, torch.Tensor] = {}

    # -- to be provided ------------------------------------------------------------------------------
    def names(self) -> Sequence[str]:
        raise NotImplementedError

    def meta(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        """(storage dtype in this run, shape)."""
        raise NotImplementedError

    def _make(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    # -- mapping -------------------------------------------------------------------------------------
    def keep(self, names: Iterable[str]) -> None:
        self._keep.update(names)

    def __contains__(self, name) -> bool:
        return name in set(self.names())

    def __iter__(self) -> Iterator[str]:
        return iter(self.names())

    def __len__(self) -> int:
        return len(self.names())

    def keys(self):
        return list(self.names())

    def items(self):
        return ((n, self[n]) for n in self.names())

    def __getitem__(self, name: str) -> torch.Tensor:
        if name in self._kept:
            return self._kept[name]
        if name not in self:
            raise KeyError(name)
        t = self._make(name)
        if name in self._keep:
            self._kept[name] = t
        return t

    def close(self) -> None:
        self._kept.clear()


def tensor_meta(tensors, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
    """dtype and shape of ``tensors[name]`` for a :class:`TensorSource` (no data read) or a plain dict."""
    meta = getattr(tensors, "meta", None)
    if meta is not None:
        return meta(name)
    t = tensors[name]
    return t.dtype, tuple(t.shape)


def fused_rows(tensors, names: Sequence[str], device: torch.device, interleave: bool = False) -> torch.Tensor:
    """The named tensors side by side along their first dimension in one buffer made for them, filled one tensor
    at a time: stacked (``[a; b; c]``), or with ``interleave`` row by row (``a0, b0, a1, b1, ...``; equal shapes).
    Tensors of different floating types meet in float32."""
    metas = [tensor_meta(tensors, n) for n in names]
    dts = {m[0] for m in metas}
    dtype = dts.pop() if len(dts) == 1 else torch.float32
    rest = metas[0][1][1:]
    if any(m[1][1:] != rest for m in metas) or (interleave and any(m[1] != metas[0][1] for m in metas)):
        raise ValueError(f"tensors {', '.join(names)} do not fit side by side")
    rows = [m[1][0] for m in metas]
    out = torch.empty((sum(rows),) + tuple(rest), dtype=dtype, device=device)
    if interleave:
        view = out.view(rows[0], len(names), *rest)
        for i, n in enumerate(names):
            view[:, i].copy_(tensors[n])
        return out
    at = 0
    for n, r in zip(names, rows):
        out[at:at + r].copy_(tensors[n])
        at += r
    return out


class _Staging:
    """Two pinned buffers through which file bytes go to the device: one is filled from the file mapping while
    the copy out of the other is in flight."""
    CHUNK = 64 << 20

    def __init__(self):
        self.bufs = [torch.empty(self.CHUNK, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        self.events = [None, None]
        self.at = 0

    def upload(self, raw: np.ndarray, device: torch.device) -> torch.Tensor:
        n = raw.shape[0]
        out = torch.empty(n, dtype=torch.uint8, device=device)
        for a in range(0, n, self.CHUNK):
            m = min(self.CHUNK, n - a)
            i = self.at
            self.at ^= 1
            if self.events[i] is not None:
                self.events[i].synchronize()
            np.copyto(self.bufs[i].numpy()[:m], raw[a:a + m])
            out[a:a + m].copy_(self.bufs[i][:m], non_blocking=True)
            self.events[i] = torch.cuda.Event()
            self.events[i].record()
        return out


class CheckpointSource(TensorSource):
    """The tensors of a model folder's safetensors files, read from the files' mappings on demand."""

    def __init__(self, folder: str, run_dtype: torch.dtype, device: torch.device):
        super().__init__(run_dtype, device)
        self.folder = folder
        paths, self.index = find_weight_files(folder)
        self.files: List[SafetensorsFile] = []
        self.where: Dict[str, SafetensorsFile] = {}
        twice: Dict[str, List[str]] = {}
        try:
            for p in paths:
                f = SafetensorsFile(p)
                self.files.append(f)
                for name in f.names():
                    if name in self.where:
                        twice.setdefault(name, [os.path.basename(self.where[name].path)]).append(os.path.basename(p))
                    else:
                        self.where[name] = f
            if twice:
                raise WeightFormatError(f"{folder}: " + "; ".join(
                    f"tensor '{n}' is in {' and '.join(fs)}" for n, fs in sorted(twice.items())))
        except WeightFormatError:
            self.close()
            raise
        self._staging: Optional[_Staging] = None

    def paths(self) -> List[str]:
        return [f.path for f in self.files]

    def names(self):
        return self.where.keys()

    def __contains__(self, name):
        return name in self.where

    def misplaced(self) -> List[str]:
        """Names the index places in a file that does not hold them."""
        if not self.index:
            return []
        return sorted(n for n, fn in self.index.items()
                      if n not in self.where or os.path.basename(self.where[n].path) != fn)

    def stored(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        f = self.where[name]
        return f.dtype(name), tuple(f.shape(name))

    def meta(self, name: str):
        dt, shape = self.stored(name)
        return storage_dtype(dt, self.run_dtype), shape

    def _make(self, name: str) -> torch.Tensor:
        f = self.where[name]
        dt, shape = self.stored(name)
        want = storage_dtype(dt, self.run_dtype)
        if self.device.type != "cuda":
            return f.tensor(name).to(want).to(self.device)
        raw = f.raw(name)
        if raw.shape[0] == 0:
            return torch.empty(shape, dtype=want, device=self.device)
        if self._staging is None:
            self._staging = _Staging()
        with torch.cuda.device(self.device):
            t = self._staging.upload(raw, self.device).view(dt).reshape(shape)
            return t if dt == want else t.to(want)       # converted on the device: the raw copy goes at once

    def close(self) -> None:
        super().close()
        if getattr(self, "_staging", None) is not None:
            for e in self._staging.events:
                if e is not None:
                    e.synchronize()
            self._staging = None
        for f in self.files:
            f.close()
        self.files, self.where = [], {}

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def check_against_specs(where: str, specs: Sequence[TensorSpec], have: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]],
                        misplaced: Sequence[str] = ()) -> None:
    """Compare a directory of stored tensors (name -> dtype, shape) with what the model declares; raise one
    :class:`WeightError` that lists every difference."""
    want = {s.name: s for s in specs}
    missing = [s.name for s in specs if s.name not in have and not s.optional]
    unexpected = sorted(set(have) - set(want))
    misshapen = [(n, have[n][1], tuple(want[n].shape)) for n in sorted(set(have) & set(want))
                 if tuple(have[n][1]) != tuple(want[n].shape)]
    other = [f"tensor '{n}' has dtype {have[n][0]}, which is neither floating nor integer"
             for n in sorted(set(have) & set(want)) if have[n][0] == torch.bool]
    other += [f"tensor '{n}' is not in the file the index names for it" for n in misplaced
              if n in want and n not in missing]
    if missing or unexpected or misshapen or other:
        raise WeightError(where, missing, unexpected, misshapen, other)


def load_tensors(folder: str, specs: Iterable[TensorSpec], run_dtype: torch.dtype,
                 device: torch.device) -> CheckpointSource:
    """Open the folder's weight files and check them against ``specs``; tensors are read when asked for."""
    specs = list(specs)
    src = CheckpointSource(folder, run_dtype, device)
    try:
        where = src.paths()[0] if len(src.files) == 1 else folder
        check_against_specs(where, specs, {n: src.stored(n) for n in src.names()}, src.misplaced())
    except WeightError:
        src.close()
        raise
    return src
