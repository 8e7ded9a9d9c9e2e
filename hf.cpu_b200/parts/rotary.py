"""Rotary position encoding with half-split pairing.

Angles ``pos * theta^(-2i/n_rot)`` for i < n_rot/2; the pair (i, i + n_rot/2) of each head is
rotated: ``a' = a*cos - b*sin``, ``b' = a*sin + b*cos``; dimensions >= n_rot are untouched
(src/model.c:468-493; pairing fixed by ``rope_neox`` for this architecture, src/model.c:140).
The table of cos/sin is computed once in float64 and rounded to float32, as the reference
evaluates cos and sin in double (src/mathx.c:92-113).
"""
from __future__ import annotations

import torch

from ..config.base import UnsupportedError
from .base import PositionEncoding, register_part


class Rotary(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, n_rot: int, theta: float, pairing: str = "half", **_):
        if pairing != "half":
            raise UnsupportedError(f"rotary pairing '{pairing}' is not supported (only 'half')")
        if n_rot % 2 or n_rot > head_dim or n_rot < 2:
            raise UnsupportedError(f"rotary width {n_rot} must be even and at most head_dim {head_dim}")
        self.head_dim, self.n_rot, self.theta = int(head_dim), int(n_rot), float(theta)
        self.cos_sin = None     # float32 [positions, n_rot/2, 2]

    def prepare(self, max_positions, device):
        half = self.n_rot // 2
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                        -2.0 * torch.arange(half, dtype=torch.float64) / self.n_rot)
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos_sin = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).contiguous().to(device)


register_part("position", "rotary", Rotary)
