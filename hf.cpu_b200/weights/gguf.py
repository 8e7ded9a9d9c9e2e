"""The reference's own model file format, GGUF, for float tensor types only (F32, F16, BF16).

This file knows the container, not the model: header, metadata key/values, tensor directory, aligned data
section.  What the metadata keys mean and what the tensors are called is the architecture's business: the
configuration class found in the registry under ``general.architecture`` turns metadata into a typed
configuration (``from_gguf``) and gives the table from checkpoint names to the file's tensor names
(``gguf_names``), as the reference's loader does per architecture (src/model.c:107-184).

Dimensions are stored innermost first (``ne[0]`` = columns, src/model.h:18-19).  The file is mapped, not
read (src/pal.c:33-52); every offset and count is checked against the file size before any data is touched,
as the reference's reader does (src/gguf.c:178-259).  Quantised tensor types are refused.
"""
from __future__ import annotations

import mmap
import os
import struct
from typing import Any, Dict, Iterable, List, Sequence, Tuple

import numpy as np
import torch

from .loader import TensorSource, check_against_specs, storage_dtype
from .safetensors_io import WeightFormatError

_TYPES = {0: (torch.float32, 4), 1: (torch.float16, 2), 30: (torch.bfloat16, 2)}
_TYPE_ID = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}
_ALIGN = 32
# metadata value types of the format
U32, F32, STRING = 4, 6, 8

TYPE_NAMES = {0: "F32", 1: "F16", 30: "BF16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K",
              11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 15: "Q8_K"}
KV_TYPE_NAMES = {0: "u8", 1: "i8", 2: "u16", 3: "i16", 4: "u32", 5: "i32", 6: "f32", 7: "bool", 8: "string", 9: "array",
                 10: "u64", 11: "i64", 12: "f64"}


def _str(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


class _Reader:
    def __init__(self, data, path: str):
        self.d, self.p, self.path = data, 0, path

    def take(self, fmt: str):
        n = struct.calcsize(fmt)
        if self.p + n > len(self.d):
            raise WeightFormatError(f"{self.path}: truncated at byte {self.p}")
        v = struct.unpack_from(fmt, self.d, self.p)
        self.p += n
        return v[0] if len(v) == 1 else v

    def string(self) -> str:
        n = self.take("<Q")
        if n > len(self.d) - self.p:
            raise WeightFormatError(f"{self.path}: string of {n} bytes at byte {self.p} exceeds the file")
        s = bytes(self.d[self.p:self.p + n])
        self.p += n
        return s.decode("utf-8", "replace")

    _SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}

    def value(self, t: int, depth: int = 0):
        if t in self._SCALAR:
            return self.take(self._SCALAR[t])
        if t == 8:
            return self.string()
        if t == 9 and depth == 0:
            et, n = self.take("<I"), self.take("<Q")
            if n > len(self.d) - self.p:
                raise WeightFormatError(f"{self.path}: array of {n} elements at byte {self.p} exceeds the file")
            return [self.value(et, 1) for _ in range(n)]
        raise WeightFormatError(f"{self.path}: unknown metadata type {t} at byte {self.p}")


def parse_gguf(data, path: str):
    """The file's directory without its tensor data: (version, metadata {key: value}, metadata types {key: type id},
    tensor infos [(name, dims innermost first, type id, offset)], alignment, offset of the data section).
    ``data`` is the file's bytes or a memory map of it."""
    r = _Reader(data, path)
    if bytes(data[:4]) != b"GGUF":
        raise WeightFormatError(f"{path}: not a GGUF file")
    r.p = 4
    version, n_tensors, n_kv = r.take("<I"), r.take("<Q"), r.take("<Q")
    if version not in (2, 3):
        raise WeightFormatError(f"{path}: GGUF version {version} is not supported")
    if n_tensors > len(data) or n_kv > len(data):
        raise WeightFormatError(f"{path}: counts exceed the file size")
    meta, kinds = {}, {}
    for _ in range(n_kv):
        key = r.string()
        kinds[key] = r.take("<I")
        meta[key] = r.value(kinds[key])
    infos = []
    for _ in range(n_tensors):
        name = r.string()
        nd = r.take("<I")
        if nd > 4:
            raise WeightFormatError(f"{path}: tensor '{name}' has {nd} dimensions")
        dims = [r.take("<Q") for _ in range(nd)]
        infos.append((name, dims, r.take("<I"), r.take("<Q")))
    align = int(meta.get("general.alignment", _ALIGN)) or _ALIGN
    base = (r.p + align - 1) // align * align
    return version, meta, kinds, infos, align, base


class GgufFile:
    """A mapped GGUF file: metadata and the tensor directory, tensors by the file's own names on demand."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except FileNotFoundError:
            raise WeightFormatError(f"{path}: no such file") from None
        self._mm = None
        try:
            size = os.fstat(self._f.fileno()).st_size
            if size == 0:
                raise WeightFormatError(f"{path}: empty file")
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
            self.version, self.meta, self.kinds, self.infos, self.align, self.base = parse_gguf(self._mm, path)
            self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
            for name, dims, tid, off in self.infos:
                if name in self.entries:
                    raise WeightFormatError(f"{path}: tensor '{name}' appears twice")
                if tid not in _TYPES:
                    raise WeightFormatError(f"{path}: tensor '{name}' has type {TYPE_NAMES.get(tid, tid)}; only F32, "
                                            f"F16 and BF16 are supported")
                dt, esz = _TYPES[tid]
                count = 1
                for d in dims:
                    count *= d
                if self.base + off + count * esz > size:
                    raise WeightFormatError(f"{path}: tensor '{name}' runs past the end of the file")
                self.entries[name] = (dt, tuple(reversed(dims)), self.base + off, count * esz)
        except WeightFormatError:
            self.close()
            raise

    def names(self):
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        """Outermost dimension first ([rows, columns] for a matrix)."""
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def raw(self, name: str) -> np.ndarray:
        _, _, at, nbytes = self.entries[name]
        if nbytes == 0:
            return np.empty(0, dtype=np.uint8)
        return np.frombuffer(self._mm, dtype=np.uint8, count=nbytes, offset=at)

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, _, nbytes = self.entries[name]
        if nbytes == 0:
            return torch.empty(shape, dtype=dt)
        return torch.from_numpy(self.raw(name).copy()).view(dt).reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_gguf_file(path: str, kv: Sequence[Tuple[str, int, Any]], tensors) -> None:
    """Write a version-3 file: ``kv`` = (key, value type, value) with types ``U32``, ``F32`` and ``STRING``;
    ``tensors`` = (name in the file, tensor) pairs, or (name, dtype, shape, function returning the tensor) so that
    the directory can be written before any tensor is made; data is streamed in the order given."""
    head = b""
    for key, t, v in kv:
        if t not in (U32, F32, STRING):
            raise WeightFormatError(f"metadata key '{key}': value type {t} cannot be written here")
        head += _str(key) + struct.pack("<I", t)
        head += _str(v) if t == STRING else struct.pack("<I" if t == U32 else "<f", v)
    entries = []
    for e in tensors:
        if len(e) == 2:
            name, t = e
            entries.append((name, t.dtype, tuple(t.shape), (lambda t=t: t)))
        else:
            entries.append(tuple(e))
    infos, off, places = b"", 0, []
    for name, dtype, shape, _ in entries:
        if dtype not in _TYPE_ID:
            raise WeightFormatError(f"tensor '{name}': dtype {dtype} cannot be stored in GGUF here")
        off += -off % _ALIGN
        dims = list(reversed(shape))
        infos += _str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", _TYPE_ID[dtype], off)
        nbytes = _TYPES[_TYPE_ID[dtype]][1]
        for d in shape:
            nbytes *= int(d)
        places.append((off, nbytes))
        off += nbytes
    out = b"GGUF" + struct.pack("<IQQ", 3, len(entries), len(kv)) + head + infos
    out += b"\0" * (-len(out) % _ALIGN)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(out)
        at = 0
        for (name, dtype, shape, get), (place, nbytes) in zip(entries, places):
            f.write(b"\0" * (place - at))
            t = get().detach().cpu().contiguous()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise WeightFormatError(f"tensor '{name}' is not what its directory entry says")
            if nbytes:
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
            at = place + nbytes
    os.replace(tmp, path)


def write_gguf(path: str, config, tensors, name: str = "hfb200 export") -> None:
    """Export a model: ``config`` is a configuration (or a config.json dict) whose class knows the format's
    metadata keys and tensor names for its architecture; ``tensors`` carry checkpoint names (a dict, or a source that
    makes each tensor when it is asked for).  Tensors the architecture's table leaves out (a tied head's copy) are
    not written."""
    from ..config import config_from_dict
    from .loader import tensor_meta
    cfg = config if hasattr(config, "gguf_names") else config_from_dict(config)
    table = cfg.gguf_names()
    unknown = sorted(n for n in tensors.keys() if n not in table and n not in cfg.gguf_left_out())
    if unknown:
        raise WeightFormatError(f"no GGUF name for tensor(s) {', '.join(unknown)} in architecture '{cfg.gguf_architecture}'")
    kv = [("general.architecture", STRING, cfg.gguf_architecture), ("general.name", STRING, name)] + list(cfg.gguf_metadata())
    write_gguf_file(path, kv, [(table[n],) + tensor_meta(tensors, n) + ((lambda n=n: tensors[n]),)
                               for n in tensors.keys() if n in table])


class GgufSource(TensorSource):
    """The tensors of a GGUF file under their checkpoint names, read from the mapping on demand; ``config`` is the
    configuration its metadata describe."""

    def __init__(self, path: str, run_dtype: torch.dtype, device: torch.device):
        super().__init__(run_dtype, device)
        from ..config import config_from_gguf
        self.file = GgufFile(path)
        try:
            self.config = config_from_gguf(self.file.meta, {n: self.file.shape(n) for n in self.file.names()}, path)
            back = {g: c for c, g in self.config.gguf_names().items()}
            self.where = {back.get(n, n): n for n in self.file.names()}
        except Exception:
            self.file.close()
            raise
        self._staging = None

    def names(self):
        return self.where.keys()

    def __contains__(self, name):
        return name in self.where

    def stored(self, name):
        g = self.where[name]
        return self.file.dtype(g), self.file.shape(g)

    def meta(self, name):
        dt, shape = self.stored(name)
        return storage_dtype(dt, self.run_dtype), shape

    def _make(self, name):
        dt, shape = self.stored(name)
        want = storage_dtype(dt, self.run_dtype)
        if self.device.type != "cuda":
            return self.file.tensor(self.where[name]).to(want).to(self.device)
        raw = self.file.raw(self.where[name])
        if raw.shape[0] == 0:
            return torch.empty(shape, dtype=want, device=self.device)
        from .loader import _Staging
        if self._staging is None:
            self._staging = _Staging()
        with torch.cuda.device(self.device):
            t = self._staging.upload(raw, self.device).view(dt).reshape(shape)
            return t if dt == want else t.to(want)

    def check(self, specs) -> None:
        check_against_specs(self.file.path, list(specs), {n: self.stored(n) for n in self.names()})

    def close(self):
        super().close()
        if self._staging is not None:
            for e in self._staging.events:
                if e is not None:
                    e.synchronize()
            self._staging = None
        self.file.close()


def read_gguf(path: str):
    """(configuration, {checkpoint name: CPU tensor}) of a whole file; for tools and tests, the engine loads
    through :class:`GgufSource`."""
    src = GgufSource(path, torch.float32, torch.device("cpu"))
    try:
        return src.config, {n: src.file.tensor(src.where[n]) for n in src.names()}
    finally:
        src.close()
