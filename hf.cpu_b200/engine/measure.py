"""The arithmetic behind the reported fractions: bytes a decode step must read, operations a step performs, and
the peaks they are divided by.

``hbm_frac`` of a decode step = (every weight the step uses, once, + the cache of the live requests) / time /
the copy bandwidth; ``mma_frac`` of a prompt step = its multiply-adds x 2 / time / the dense bfloat16 peak.  The
peaks are the ones measured on this machine when a ``MEASURED_PEAKS.json`` is at hand, else stated fallbacks.
The reference reports tokens a second only (src/ops.c:1016-1023); the fractions say how far those are from what
the hardware allows.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Sequence, Tuple

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PEAKS_FILE = "MEASURED_PEAKS.json"


def load_peaks(*folders: str) -> Tuple[Dict[str, float], str]:
    """({"hbm_gbs", "bf16_tflops"}, "measured" | "fallback"); looks for the peaks file in ``folders``, the working
    directory and the folder above the package."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    for folder in list(folders) + [os.getcwd(), here]:
        try:
            with open(os.path.join(folder, PEAKS_FILE)) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"])}, "measured"
        except (OSError, KeyError, ValueError, TypeError):
            continue
    return dict(FALLBACK_PEAKS), "fallback"


def cache_bytes_per_token(engine) -> int:
    """Bytes of keys and values one token holds over all cache groups."""
    return sum(g.page_bytes for g in engine.cache.groups) // engine.block_size


def decode_step_bytes(engine, kv_lens: Sequence[int]) -> int:
    """Bytes a step of single tokens has to read: the weights once, and the keys and values the requests see."""
    total = engine.model.weight_bytes_per_step()
    for g in engine.cache.groups:
        per_token = g.page_bytes // engine.block_size
        w = g.spec.window
        total += sum((min(n, w) if w > 0 else n) * per_token for n in kv_lens)
    return total


def step_flops(model, q_lens: Sequence[int], kv_lens: Sequence[int], logit_rows: int) -> float:
    """Floating-point operations of one step (a multiply-add counts two): the parts report their own."""
    total = 0.0
    for e in model.plan.schedule:
        layer = model.layers[e.layer]
        total += layer.mixer.flops(q_lens, kv_lens) + layer.ffn.flops(sum(q_lens))
    return total + model.head.flops(logit_rows)


def fractions(engine, *, decode_ms: float = 0.0, decode_kv_lens: Sequence[int] = (), prefill_ms: float = 0.0,
              prefill_q_lens: Sequence[int] = (), prefill_kv_lens: Sequence[int] = (), peaks=None) -> Dict[str, float]:
    pk = peaks or load_peaks()[0]
    out = {}
    if decode_ms > 0:
        out["hbm_frac"] = decode_step_bytes(engine, decode_kv_lens) / (decode_ms * 1e-3) / (pk["hbm_gbs"] * 1e9)
    if prefill_ms > 0:
        flops = step_flops(engine.model, prefill_q_lens, prefill_kv_lens or prefill_q_lens, len(prefill_q_lens))
        out["mma_frac"] = flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
    return out
