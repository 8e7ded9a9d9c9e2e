"""Host mirror of the sampler, and log-probabilities.

The order of operations is the reference's (src/sample.c:66-116): greedy takes the first index of the
maximum; otherwise candidates are ordered by logit (ties: lower id first), cut to top-k, turned into
probabilities ``exp((l - max)/temp) / sum``, cut by min-p (``p >= min_p * p_max``, at least one), cut by
top-p (smallest prefix whose cumulative probability reaches it), and one is drawn with
``r = u * sum(kept)``: the first candidate whose cumulative sum exceeds r.  All sums are float32 and
sequential, as in the reference.
"""
from __future__ import annotations

import math
from typing import List, Tuple

import numpy as np

from .params import SamplingParams
from .rng import Rng


def sample_host(logits: np.ndarray, p: SamplingParams, rng: Rng) -> int:
    l = np.asarray(logits, dtype=np.float32)
    if p.temp <= 0:
        return int(np.argmax(l))
    n = len(l)
    if 0 < p.top_k < n:
        part = np.argpartition(-l, p.top_k - 1)[:p.top_k]
        kth = l[part].min()
        cand = np.nonzero(l >= kth)[0]             # includes every tie of the k-th value
        order = cand[np.lexsort((cand, -l[cand]))][:p.top_k]
    else:
        order = np.lexsort((np.arange(n), -l))
    probs = np.exp(((l[order] - l[order[0]]) / np.float32(p.temp)).astype(np.float32)).astype(np.float32)
    probs = (probs / _seq_sum(probs)).astype(np.float32)
    kept = len(probs)
    if p.min_p > 0:
        thr = np.float32(p.min_p) * probs[0]
        below = np.nonzero(probs < thr)[0]
        kept = max(int(below[0]) if len(below) else len(probs), 1)
    if 0 < p.top_p < 1:
        cum = np.cumsum(probs[:kept], dtype=np.float32)
        hit = np.nonzero(cum >= np.float32(p.top_p))[0]
        if len(hit):
            kept = int(hit[0]) + 1
    cum = np.cumsum(probs[:kept], dtype=np.float32)
    r = np.float32(rng.uniform() * cum[-1])
    hit = np.nonzero(r < cum)[0]
    return int(order[int(hit[0])] if len(hit) else order[kept - 1])


def _seq_sum(x: np.ndarray) -> np.float32:
    return np.cumsum(x, dtype=np.float32)[-1]


def logprob(logits: np.ndarray, tok: int) -> float:
    """``l_tok - max - log(sum exp(l - max))`` with the sum in double (src/sample.c:25-33)."""
    l = np.asarray(logits, dtype=np.float32)
    mx = l.max()
    return float(np.float64(l[tok] - mx) - math.log(np.exp((l - mx).astype(np.float32)).astype(np.float64).sum()))


def top_logprobs(logits: np.ndarray, k: int) -> List[Tuple[int, float]]:
    """The k best (id, logprob), k at most 64, ties by lower id (src/sample.c:35-55)."""
    l = np.asarray(logits, dtype=np.float32)
    k = min(k, 64, len(l))
    mx = l.max()
    lse = math.log(np.exp((l - mx).astype(np.float32)).astype(np.float64).sum())
    order = np.lexsort((np.arange(len(l)), -l))[:k]
    return [(int(i), float(np.float32(np.float64(l[i] - mx) - lse))) for i in order]
