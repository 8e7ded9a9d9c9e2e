"""Sampling on the device: per-row parameters go up, token ids come back.

The generator stays on the host (it is a few integer operations per token, src/sample.c:15-23): each
non-greedy row's next draw is computed here and passed to the kernel, so a request's sequence of
draws does not depend on batching or on preemption.
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from .. import kernels


def sample_rows(logits: torch.Tensor, reqs) -> List[int]:
    """``reqs[i]`` (with ``.params`` and ``.rng``) owns row i of the float32 ``logits`` [M, V]."""
    M = logits.shape[0]
    if all(r.params.temp <= 0 for r in reqs):
        out = torch.empty(M, dtype=torch.int32, device=logits.device)
        kernels.argmax(logits.contiguous(), out)             # greedy rows need no parameters and no draws
        return out.tolist()
    host = np.zeros((5, M), dtype=np.float32)
    for i, r in enumerate(reqs):
        p = r.params
        host[0, i], host[2, i], host[3, i] = p.temp, p.top_p, p.min_p
        host[1, i] = np.int32(p.top_k).view(np.float32)
        host[4, i] = r.rng.uniform() if p.temp > 0 else 0.0
    dev = torch.from_numpy(host).to(logits.device, non_blocking=True)
    out = torch.empty(M, dtype=torch.int32, device=logits.device)
    kernels.sample(logits.contiguous(), dev[0], dev[1].view(torch.int32), dev[2], dev[3], dev[4], out)
    return out.tolist()
