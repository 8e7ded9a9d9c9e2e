"""The reference's own model file format, GGUF, for float types only (F32, F16, BF16).

Reads and writes version 3 files with the tensor names and metadata keys the reference's loader uses
(src/model.c:107-184): ``general.architecture``, ``<arch>.block_count``, ``.embedding_length``,
``.feed_forward_length``, ``.attention.head_count``, ``.attention.head_count_kv``, ``.attention.key_length``,
``.attention.layer_norm_rms_epsilon``, ``.rope.freq_base``, ``.context_length``; tensors ``token_embd.weight``,
``output_norm.weight``, ``output.weight`` (absent = tied head), ``blk.N.attn_{q,k,v}.{weight,bias}``,
``blk.N.attn_output.weight``, ``blk.N.attn_norm.weight``, ``blk.N.ffn_norm.weight``, ``blk.N.ffn_{gate,up,down}.weight``.
Dimensions are stored innermost first (``ne[0]`` = columns, src/model.h:18-19).  Every offset and count is
checked against the file size, as the reference's reader does (src/gguf.c:178-259).  Quantised tensor types
are refused.
"""
from __future__ import annotations

import re
import struct
from typing import Any, Dict, Tuple

import numpy as np
import torch

from .safetensors_io import WeightFormatError

_TYPES = {0: (torch.float32, 4), 1: (torch.float16, 2), 30: (torch.bfloat16, 2)}
_TYPE_ID = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}
_ALIGN = 32

_LAYER_NAMES = {
    "attn_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight",
    "attn_v.weight": "self_attn.v_proj.weight", "attn_output.weight": "self_attn.o_proj.weight",
    "attn_q.bias": "self_attn.q_proj.bias", "attn_k.bias": "self_attn.k_proj.bias", "attn_v.bias": "self_attn.v_proj.bias",
    "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight", "ffn_down.weight": "mlp.down_proj.weight",
}
_TOP_NAMES = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
              "output.weight": "lm_head.weight"}


def to_checkpoint_name(gguf_name: str) -> str:
    if gguf_name in _TOP_NAMES:
        return _TOP_NAMES[gguf_name]
    m = re.fullmatch(r"blk\.(\d+)\.(.+)", gguf_name)
    if m and m.group(2) in _LAYER_NAMES:
        return f"model.layers.{m.group(1)}.{_LAYER_NAMES[m.group(2)]}"
    return gguf_name


def to_gguf_name(name: str) -> str:
    for k, v in _TOP_NAMES.items():
        if v == name:
            return k
    m = re.fullmatch(r"model\.layers\.(\d+)\.(.+)", name)
    if m:
        for k, v in _LAYER_NAMES.items():
            if v == m.group(2):
                return f"blk.{m.group(1)}.{k}"
    return name


def _str(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, config: Dict[str, Any], tensors: Dict[str, torch.Tensor], arch: str = "qwen2") -> None:
    """``config`` is a config.json dict; ``tensors`` carry checkpoint names."""
    H = config["num_attention_heads"]
    kv = [("general.architecture", 8, arch), ("general.name", 8, "hfb200 export"),
          (f"{arch}.block_count", 4, config["num_hidden_layers"]),
          (f"{arch}.context_length", 4, config.get("max_position_embeddings", 0)),
          (f"{arch}.embedding_length", 4, config["hidden_size"]),
          (f"{arch}.feed_forward_length", 4, config["intermediate_size"]),
          (f"{arch}.attention.head_count", 4, H),
          (f"{arch}.attention.head_count_kv", 4, config.get("num_key_value_heads", H)),
          (f"{arch}.attention.key_length", 4, config.get("head_dim") or config["hidden_size"] // H),
          (f"{arch}.attention.layer_norm_rms_epsilon", 6, config.get("rms_norm_eps", 1e-5)),
          (f"{arch}.rope.freq_base", 6, config.get("rope_theta", 10000.0))]
    head = b""
    for key, t, v in kv:
        head += _str(key) + struct.pack("<I", t)
        head += _str(v) if t == 8 else struct.pack("<I" if t == 4 else "<f", v)
    infos, blob = b"", b""
    names = [n for n in tensors if not (n == "lm_head.weight" and config.get("tie_word_embeddings"))]
    for name in names:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TYPE_ID:
            raise WeightFormatError(f"tensor '{name}': dtype {t.dtype} cannot be stored in GGUF here")
        blob += b"\0" * (-len(blob) % _ALIGN)
        dims = list(reversed(t.shape))
        infos += _str(to_gguf_name(name)) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", _TYPE_ID[t.dtype], len(blob))
        blob += t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes()
    out = b"GGUF" + struct.pack("<IQQ", 3, len(names), len(kv)) + head + infos
    out += b"\0" * (-len(out) % _ALIGN)
    with open(path, "wb") as f:
        f.write(out + blob)


class _Reader:
    def __init__(self, data: bytes, path: str):
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
        s = self.d[self.p:self.p + n]
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


TYPE_NAMES = {0: "F32", 1: "F16", 30: "BF16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K",
              11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 15: "Q8_K"}
KV_TYPE_NAMES = {0: "u8", 1: "i8", 2: "u16", 3: "i16", 4: "u32", 5: "i32", 6: "f32", 7: "bool", 8: "string", 9: "array",
                 10: "u64", 11: "i64", 12: "f64"}


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


def read_gguf(path: str) -> Tuple[Dict[str, Any], Dict[str, torch.Tensor]]:
    """Returns (config.json-style dict, tensors by checkpoint name)."""
    try:
        data = open(path, "rb").read()
    except FileNotFoundError:
        raise WeightFormatError(f"{path}: no such file") from None
    version, meta, _, infos, align, base = parse_gguf(data, path)
    tensors, seen = {}, set()
    for name, dims, tid, off in infos:
        if name in seen:
            raise WeightFormatError(f"{path}: tensor '{name}' appears twice")
        seen.add(name)
        if tid not in _TYPES:
            raise WeightFormatError(f"{path}: tensor '{name}' has type {tid}; only F32, F16 and BF16 are supported")
        dt, esz = _TYPES[tid]
        count = 1
        for d in dims:
            count *= d
        if base + off + count * esz > len(data):
            raise WeightFormatError(f"{path}: tensor '{name}' runs past the end of the file")
        raw = np.frombuffer(data, dtype=np.uint8, count=count * esz, offset=base + off).copy()
        tensors[to_checkpoint_name(name)] = torch.from_numpy(raw).view(dt).reshape(list(reversed(dims)))
    arch = meta.get("general.architecture")
    if not isinstance(arch, str):
        raise WeightFormatError(f"{path}: general.architecture is missing")

    def need(key):
        if f"{arch}.{key}" not in meta:
            raise WeightFormatError(f"{path}: metadata key '{arch}.{key}' is missing")
        return meta[f"{arch}.{key}"]
    E, H = need("embedding_length"), need("attention.head_count")
    if "model.embed_tokens.weight" not in tensors:
        raise WeightFormatError(f"{path}: tensor 'token_embd.weight' is missing")
    cfg = {"model_type": arch, "num_hidden_layers": need("block_count"), "hidden_size": E,
           "intermediate_size": need("feed_forward_length"), "num_attention_heads": H,
           "num_key_value_heads": meta.get(f"{arch}.attention.head_count_kv", H),
           "head_dim": meta.get(f"{arch}.attention.key_length", E // H if H else 0),
           "rms_norm_eps": float(meta.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5)),
           "rope_theta": float(meta.get(f"{arch}.rope.freq_base", 10000.0)),
           "max_position_embeddings": meta.get(f"{arch}.context_length", 0) or 32768,
           "vocab_size": tensors["model.embed_tokens.weight"].shape[0],
           "tie_word_embeddings": "lm_head.weight" not in tensors}
    return cfg, tensors
