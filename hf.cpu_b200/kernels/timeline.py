"""The kernel timeline of a build with ``-DHFB_TRACE`` (developers): where a step's time goes, kernel by kernel.

In such a build (``HFB_NVCC_EXTRA=-DHFB_TRACE`` in the environment when the library is built) thread 0 of block 0 of
every kernel logs ``%globaltimer`` when the block starts ("entry") and when its wait for the kernel in front returns
("ready"); a few kernels log further marks.  Every kernel is launched so that it may start while its predecessor
still runs, so a kernel's own time is the span from its "ready" to its successor's "ready" ("busy"), and "early" is
how long it was resident before it could begin.  The reference accounts for a step per phase with wall-clock
accumulators (src/model.h:75-79, results/hp-profile-q8_0-n1.txt); this is the same question asked of the device.
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

from . import backend

KERNELS = {1: "gemm", 2: "rope_kv", 3: "attn_decode", 4: "attn_merge", 5: "reduce_norm", 6: "rmsnorm", 7: "embed",
           8: "splitk_reduce", 9: "argmax_chunks", 10: "argmax_final", 11: "reduce_norm_scalar", 12: "attn_fast",
           13: "attn_tc", 14: "swiglu", 15: "rmsnorm_s", 16: "rope_kv_write"}
MARKS = {0: "entry", 1: "ready", 2: "setup", 3: "issued", 4: "block0_done", 5: "q_in", 6: "tiles_done", 7: "partial_stored",
         8: "last_cta_start", 9: "last_cta_end"}
CAPACITY = 32768


def start() -> None:
    """Start (or restart) logging; raises when the library was built without ``-DHFB_TRACE``."""
    lib = backend().lib
    if lib.hfb_trace_start() != 0:
        raise RuntimeError(lib.hfb_last_error().decode())


def take() -> List[Tuple[int, int, int]]:
    """The log so far as (nanoseconds, kernel id or 0, mark) sorted by time; clears it."""
    lib = backend().lib
    lib.hfb_trace_take.restype = ctypes.c_longlong
    buf = (ctypes.c_ulonglong * (2 * CAPACITY))()
    n = lib.hfb_trace_take(buf, ctypes.c_longlong(CAPACITY))
    return sorted((int(buf[2 * i + 1]), int(buf[2 * i] >> 8), int(buf[2 * i] & 255)) for i in range(n))


def kernels(records) -> List[dict]:
    """One row per kernel: name, entry, ready, busy (until the successor's ready) and early, in microseconds from the
    first entry."""
    entries = [(t, k) for t, k, m in records if m == 0]
    readies = [t for t, k, m in records if m == 1]
    if not entries:
        return []
    t0 = entries[0][0]
    rows, prev = [], -1
    for t, k in entries:
        later = [r for r in readies if r >= t and r > prev]
        ready = later[0] if later else t
        prev = ready
        rows.append({"kernel": KERNELS.get(k, str(k)), "entry": (t - t0) / 1e3, "ready": (ready - t0) / 1e3})
    for i, row in enumerate(rows):
        end = rows[i + 1]["ready"] if i + 1 < len(rows) else row["ready"]
        row["busy"], row["early"] = end - row["ready"], row["ready"] - row["entry"]
    return rows


def format_rows(rows) -> str:
    return "\n".join(f"{i:3d} {r['kernel']:18s} entry {r['entry']:9.2f}  ready {r['ready']:9.2f}  early {r['early']:6.2f}  "
                     f"busy {r['busy']:7.2f}" for i, r in enumerate(rows))


def format_marks(records) -> str:
    t0 = records[0][0] if records else 0
    return "\n".join(f"{(t - t0) / 1e3:9.2f}  {MARKS.get(m, str(m)):15s} {KERNELS.get(k, '') if m == 0 else ''}"
                     for t, k, m in records)
