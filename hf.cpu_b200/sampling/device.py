"""Sampling on the device: per-row parameters go up, token ids come back.

The generator stays on the host (it is a few integer operations per token, src/sample.c:15-23): each
non-greedy row's next draw is computed here and passed to the kernel, so a request's sequence of
draws does not depend on batching or on preemption.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from .. import kernels


class Pending:
    """Token ids a sampling kernel is writing: ``device`` holds them for a step that runs ahead of the host,
    ``tokens()`` waits for the copy to the host and returns them."""

    def __init__(self, device: torch.Tensor, host: Optional[torch.Tensor] = None):
        self.device = device
        n = device.numel()
        # ``host``: a pinned buffer of the caller's (one slot longer than the ids) that stays untouched until
        # tokens() has returned; its last slot receives the device error word as it stands after this step
        if host is None or host.numel() < n + 1:
            host = torch.empty(n + 1, dtype=device.dtype, pin_memory=True)
        self._host, self._word = host[:n], host[n:n + 1]
        self._host.copy_(device, non_blocking=True)
        b = kernels.backend()
        self._checked = hasattr(b, "error_word_async")
        if self._checked:
            b.error_word_async(self._word)
        self._event = torch.cuda.Event()
        self._event.record()

    def tokens(self) -> List[int]:
        """The ids, once they are on the host.  Raises :class:`kernels.DeviceFault` when a kernel of this step (or
        of one before it, since the last look) recorded an error: the ids are then worthless."""
        self._event.synchronize()
        if self._checked and int(self._word[0]) != 0:
            word = int(self._word[0])
            try:
                kernels.check_device_errors()          # reads the word again and clears it
            except kernels.DeviceFault:
                pass
            raise kernels.DeviceFault(word)
        return self._host.tolist()


def launch_rows(logits: torch.Tensor, reqs) -> torch.Tensor:
    """Launches the sampling of ``reqs[i]`` (with ``.params`` and ``.rng``) from row i of the float32 ``logits``
    [M, V]; returns the int32 token ids on the device."""
    M = logits.shape[0]
    out = torch.empty(M, dtype=torch.int32, device=logits.device)
    if all(r.params.temp <= 0 for r in reqs):
        kernels.argmax(logits.contiguous(), out)             # greedy rows need no parameters and no draws
        return out
    host = np.zeros((5, M), dtype=np.float32)
    for i, r in enumerate(reqs):
        p = r.params
        host[0, i], host[2, i], host[3, i] = p.temp, p.top_p, p.min_p
        host[1, i] = np.int32(p.top_k).view(np.float32)
        host[4, i] = r.rng.uniform() if p.temp > 0 else 0.0
    dev = torch.from_numpy(host).to(logits.device, non_blocking=True)
    kernels.sample(logits.contiguous(), dev[0], dev[1].view(torch.int32), dev[2], dev[3], dev[4], out)
    return out


def sample_rows_async(logits: torch.Tensor, reqs, host: Optional[torch.Tensor] = None) -> Pending:
    return Pending(launch_rows(logits, reqs), host)


def sample_rows(logits: torch.Tensor, reqs) -> List[int]:
    """``reqs[i]`` (with ``.params`` and ``.rng``) owns row i of the float32 ``logits`` [M, V]."""
    return launch_rows(logits, reqs).tolist()
