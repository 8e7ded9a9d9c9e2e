"""A small reader and writer for the safetensors container.

Layout: 8 bytes little-endian header length N, N bytes of JSON mapping each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets are
relative to the first byte after the header), then the raw little-endian data.
The reference has no such reader (it reads GGUF, src/gguf.c); the checks here
mirror its hardening: sizes and offsets are bounded by the file (src/gguf.c:191-259).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch


class WeightFormatError(ValueError):
    """The file is not a well-formed safetensors container."""


_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """Read-only view of one file; tensors are materialised one at a time."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except FileNotFoundError:
            raise WeightFormatError(f"{path}: no such file") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightFormatError(f"{path}: file has {size} bytes, too short for a safetensors header")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8 or n > 1 << 30:
            raise WeightFormatError(f"{path}: header length {n} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFormatError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise WeightFormatError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {})
        self._data0 = 8 + n
        self._size = size
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise WeightFormatError(f"{path}: malformed entry for tensor '{name}'") from None
            if dt not in _DTYPES:
                raise WeightFormatError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            tdt, esz = _DTYPES[dt]
            count = 1
            for s in shape:
                if s < 0:
                    raise WeightFormatError(f"{path}: tensor '{name}' has a negative extent")
                count *= s
            if not (0 <= b <= en <= size - self._data0) or en - b != count * esz:
                raise WeightFormatError(f"{path}: tensor '{name}' data [{b}, {en}) does not match shape "
                                        f"{list(shape)} of {dt} within a file of {size} bytes")
            self.entries[name] = (tdt, shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def raw(self, name: str) -> np.ndarray:
        """The named tensor's bytes as a read-only view of the file mapping (nothing is copied)."""
        _, _, b, en = self.entries[name]
        if en == b:
            return np.empty(0, dtype=np.uint8)
        return np.frombuffer(self._mm, dtype=np.uint8, count=en - b, offset=self._data0 + b)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor holding a copy of the named tensor's data."""
        tdt, shape, b, en = self.entries[name]
        if en == b:
            return torch.empty(shape, dtype=tdt)
        return torch.from_numpy(self.raw(name).copy()).view(tdt).reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:          # a view handed out by raw() is still alive; the mapping goes with it
                pass
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_safetensors(path: str, tensors, metadata: Dict[str, str] = None) -> None:
    """Write ``tensors`` (a dict, or any mapping with ``meta(name) -> (dtype, shape)`` that makes its tensors on
    demand) to ``path``; tensors are fetched and written one at a time."""
    header = {}
    off = 0
    names = sorted(tensors.keys())
    meta = getattr(tensors, "meta", None)
    for name in names:
        dtype, shape = meta(name) if meta is not None else (tensors[name].dtype, tuple(tensors[name].shape))
        if dtype not in _NAMES:
            raise WeightFormatError(f"tensor '{name}': dtype {dtype} cannot be stored")
        nbytes = _DTYPES[_NAMES[dtype]][1]
        for s_ in shape:
            nbytes *= int(s_)
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    if metadata:
        header["__metadata__"] = metadata
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in names:
            t = tensors[name].detach().cpu().contiguous()
            b, e = header[name]["data_offsets"]
            if t.numel() * t.element_size() != e - b:
                raise WeightFormatError(f"tensor '{name}' changed between the header and the data")
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
