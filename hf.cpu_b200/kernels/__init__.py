"""The kernel interface the parts call.  One backend exists in the product: the CUDA library.

The functions here check shapes and types, refuse sizes the kernels do not take with a clear
error, and forward to the backend.  There is no CPU path: without the library or without a GPU
the first call raises.  (Tests may install a stand-in backend with :func:`set_backend` to exercise
the host-side logic on a machine without a GPU.)
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.base import UnsupportedError

_backend = None

MAX_HEAD_DIM = 256
ERROR_BITS = {1: "a token id outside the vocabulary", 2: "a block-table entry that names no page",
              4: "a cache slot outside the pool", 8: "a device-side wait that ran out",
              16: "a position outside the rotary table"}


class PhaseProfile:
    """Device time per phase of the forward pass, for ``--profile``: parts wrap their kernel calls in
    ``kernels.phase(name)``; while the profile is on, each phase is bracketed by CUDA events on the current stream
    and ``take()`` returns milliseconds per name and clears them.  Off, ``phase`` costs one attribute test.  The
    reference keeps per-phase accumulators with the same names (src/model.h:75-79, src/ops.c:593-604)."""
    NAMES = ("embed", "glue", "qkv", "attn", "wo", "gate_up", "silu", "down", "head", "quant", "sample")

    class _Null:
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    class _Span:
        def __init__(self, owner, name):
            self.owner, self.name = owner, name

        def __enter__(self):
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.a.record()
            return self

        def __exit__(self, *a):
            self.b.record()
            self.owner.spans.append((self.name, self.a, self.b))
            return False

    def __init__(self):
        self.enabled, self.spans, self._null = False, [], self._Null()

    def enable(self, on: bool) -> None:
        self.enabled = bool(on) and torch.cuda.is_available()
        self.spans = []

    def phase(self, name: str):
        return self._Span(self, name) if self.enabled else self._null

    def take(self) -> dict:
        out = {n: 0.0 for n in self.NAMES}
        if self.spans:
            torch.cuda.synchronize()
            for name, a, b in self.spans:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        self.spans = []
        return out


profile = PhaseProfile()
phase = profile.phase


def backend():
    global _backend
    if _backend is None:
        from .native import NativeBackend
        _backend = NativeBackend()
    return _backend


def set_backend(b) -> None:
    global _backend
    _backend = b


def check_head_dim(d: int) -> None:
    if d % 16 or not 16 <= d <= MAX_HEAD_DIM:
        raise UnsupportedError(f"head_dim {d} is not supported: the attention kernels take multiples of 16 "
                               f"from 16 to {MAX_HEAD_DIM}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    _need(ids.dtype == torch.int32 and ids.dim() == 1, "embed: ids must be int32 [T]")
    _need(out.dtype == torch.float32 and out.shape == (ids.shape[0], table.shape[1]), "embed: out must be float32 [T, E]")
    backend().embed(ids, table, out)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    _need(x.dtype == torch.float32 and x.dim() == 2, "rmsnorm: x must be float32 [N, E]")
    _need(w.shape == (x.shape[1],) and out.shape[1] == x.shape[1], "rmsnorm: width mismatch")
    _need(rows is None or (rows.dtype == torch.int32 and rows.shape[0] == out.shape[0]), "rmsnorm: rows must be int32 [M]")
    _need(rows is not None or out.shape[0] == x.shape[0], "rmsnorm: row count mismatch")
    backend().rmsnorm(x, w, float(eps), out, rows)


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, accumulate: bool) -> None:
    """out (=|+=) a @ w.T (+ bias); ``accumulate`` adds into a float32 ``out`` (the residual stream)."""
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "linear: inner sizes differ")
    _need(out.shape == (a.shape[0], w.shape[0]), "linear: out must be [M, N]")
    _need(bias is None or bias.shape == (w.shape[0],), "linear: bias must be [N]")
    _need(not accumulate or out.dtype == torch.float32, "linear: accumulation needs a float32 output")
    backend().linear(a, w, bias, out, bool(accumulate))


def rope_kv_write(qkv, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d) -> None:
    _need(qkv.shape[1] == (H + 2 * G) * d and q_out.shape == (qkv.shape[0], H * d), "rope_kv_write: shape mismatch")
    _need(k_cache.shape[2:] == (G, d) and v_cache.shape == k_cache.shape, "rope_kv_write: cache geometry mismatch")
    _need(k_cache.dtype == qkv.dtype == q_out.dtype, "rope_kv_write: element types differ")
    _need(n_rot == 0 or (cos_sin is not None and cos_sin.shape[1:] == (n_rot // 2, 2) and cos_sin.dtype == torch.float32),
          "rope_kv_write: cos/sin table must be float32 [positions, n_rot/2, 2]")
    backend().rope_kv_write(qkv, cos_sin, int(n_rot), positions, slots, q_out, k_cache, v_cache, H, G, d)


def attention_step_arrays(q_lens, heads_per_group: int):
    """Tile lists of a step's tokens for the tiled attention kernels, as named int32 arrays.

    A tile holds consecutive tokens of one request: its request index (``seq``), its first token's index in the
    step (``t0``) and its token count (``nt``).  The heads that share a key/value head are packed into a tile's rows
    beside the tokens, so a tile of R rows takes R // heads_per_group tokens.  Tile heights: "1" = 16 rows (a step of
    single tokens; the decode kernels), "4" = 64 rows (short portions), "8" = 128 rows and "16" = two tiles of 128
    rows per work item (portions of 64 tokens and more).  A height too small for the heads per group is left out."""
    import numpy as np
    max_q, S = max(q_lens), len(q_lens)
    heights = ["1"] if max_q == 1 else (["8", "16"] if max_q >= 64 else ["4"])
    out = {}
    for h in heights:
        per = (16 * int(h)) // heads_per_group if h != "16" else 2 * (128 // heads_per_group)
        if per < 1:
            continue
        if max_q == 1:
            seq = t0 = np.arange(S, dtype=np.int32)
            nt = np.ones(S, dtype=np.int32)
        else:
            ls, lt, ln, at = [], [], [], 0
            for s_i, n in enumerate(q_lens):
                for a in range(0, n, per):
                    ls.append(s_i)
                    lt.append(at + a)
                    ln.append(min(per, n - a))
                at += n
            seq, t0, nt = (np.asarray(x, dtype=np.int32) for x in (ls, lt, ln))
        out[h + ".seq"], out[h + ".t0"], out[h + ".nt"] = seq, t0, nt
    return out


def paged_attention(q, k_cache, v_cache, meta, ctx, H, G, d, window, scale, out, tiles=None) -> None:
    """``tiles``: the device arrays of :func:`attention_step_arrays` for this step (without them only the plain
    kernel runs)."""
    check_head_dim(d)
    _need(q.shape[1] == H * d and out.shape == q.shape, "attention: shape mismatch")
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype, "attention: element types differ")
    backend().paged_attention(q, k_cache, v_cache, meta, ctx, H, G, d, int(window), float(scale), out, tiles or {})


def swiglu(gu: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = silu(gate) * up; gate and up are the two halves of a row of ``gu``, or alternate along it."""
    _need(gu.shape == (out.shape[0], 2 * out.shape[1]) and gu.dtype == out.dtype, "swiglu: shape mismatch")
    backend().swiglu(gu, out, bool(interleaved))


def linear_swiglu(a: torch.Tensor, w: torch.Tensor, gu_buf: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(g) * u where [g0, u0, g1, u1, ...] = a @ w.T (rows of ``w`` alternate gate, up).  ``gu_buf``
    [M, 2F] is scratch for the unfused form."""
    _need(a.shape[1] == w.shape[1] and w.shape[0] == 2 * out.shape[1] and out.shape[0] == a.shape[0],
          "linear_swiglu: shape mismatch")
    _need(gu_buf.shape == (a.shape[0], w.shape[0]), "linear_swiglu: scratch must be [M, 2F]")
    backend().linear_swiglu(a, w, gu_buf, out)


def linear_residual_norm(a, w, bias, residual, norm_w, eps, xn_out) -> None:
    """residual += a @ w.T (+ bias); then, if ``xn_out`` is given, xn_out = rmsnorm(residual) * norm_w."""
    _need(a.shape[1] == w.shape[1] and residual.shape == (a.shape[0], w.shape[0]) and residual.dtype == torch.float32,
          "linear_residual_norm: shape mismatch")
    _need(xn_out is None or (xn_out.shape == residual.shape and norm_w.shape == (w.shape[0],)),
          "linear_residual_norm: norm shape mismatch")
    backend().linear_residual_norm(a, w, bias, residual, norm_w, float(eps), xn_out)


def linear_rope_kv(a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d) -> None:
    """q|k|v = a @ w.T + bias, then :func:`rope_kv_write`; ``qkv_buf`` [T, (H+2G)d] is scratch for the unfused form."""
    _need(w.shape[0] == (H + 2 * G) * d and q_out.shape == (a.shape[0], H * d), "linear_rope_kv: shape mismatch")
    _need(k_cache.shape[2:] == (G, d) and v_cache.shape == k_cache.shape and k_cache.dtype == q_out.dtype,
          "linear_rope_kv: cache geometry mismatch")
    backend().linear_rope_kv(a, w, bias, qkv_buf, cos_sin, int(n_rot), positions, slots, q_out, k_cache, v_cache, H, G, d)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32 and out.shape == (logits.shape[0],),
          "argmax: logits float32 [M, V], out int32 [M]")
    backend().argmax(logits, out)


def sample(logits, temps, top_ks, top_ps, min_ps, uniforms, out) -> None:
    """One token per row; greedy where temps <= 0, else top-k / min-p / top-p sampling with the row's draw."""
    M = logits.shape[0]
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32 and out.shape == (M,), "sample: bad logits / out")
    for t, dt in ((temps, torch.float32), (top_ks, torch.int32), (top_ps, torch.float32), (min_ps, torch.float32),
                  (uniforms, torch.float32)):
        _need(t.dtype == dt and t.shape == (M,), "sample: per-row parameters must be [M]")
    backend().sample(logits, temps, top_ks, top_ps, min_ps, uniforms, out)


class DeviceFault(RuntimeError):
    """A kernel recorded an error in the device error word; what it computed is not to be trusted."""

    def __init__(self, word: int):
        self.word = int(word)
        super().__init__("a kernel met " + "; ".join(v for k, v in ERROR_BITS.items() if word & k))


def check_device_errors() -> None:
    """Raise if any kernel recorded an error since the last check (synchronises the stream)."""
    b = backend()
    word = b.error_word() if hasattr(b, "error_word") else 0
    if word:
        raise DeviceFault(word)
