"""Dense SwiGLU feed-forward: ``h = silu(x Wg^T) * (x Wu^T)``; ``out = h Wd^T`` added to the
residual; no biases (src/model.c:612-623, src/mathx.c:34).  Gate and up are one matrix product
over the concatenated rows, as the reference serves both with one pass over the activations
(src/model.c:612-615)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec, fused_rows
from .base import FeedForward, register_part


class SwiGlu(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str, names=None, **_):
        self.E, self.F = int(hidden_size), int(intermediate_size)
        n = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        return [TensorSpec(self.names["gate"], (self.F, self.E)), TensorSpec(self.names["up"], (self.F, self.E)),
                TensorSpec(self.names["down"], (self.E, self.F))]

    def bind(self, tensors, run_dtype, device):
        # rows alternate gate_i, up_i, so that a product's epilogue finds both of a pair side by side
        self.w_gate_up = fused_rows(tensors, [self.names["gate"], self.names["up"]], device, interleave=True)
        self.w_down = tensors[self.names["down"]].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def flops(self, rows):
        return 2.0 * rows * (self.w_gate_up.numel() + self.w_down.numel())

    def _hidden(self, ctx, xn):
        T = xn.shape[0]
        gu = ctx.buf("ffn_gate_up", (T, 2 * self.F), xn.dtype)
        h = ctx.buf("ffn_h", (T, self.F), xn.dtype)
        with kernels.phase("gate_up"):
            kernels.linear_swiglu(xn, self.w_gate_up, gu, h)
        return h

    def forward(self, ctx, xn, residual):
        h = self._hidden(ctx, xn)
        with kernels.phase("down"):
            kernels.linear(h, self.w_down, None, residual, accumulate=True)

    def forward_then_norm(self, ctx, xn, residual, norm, out):
        args = norm.fused_args()
        if args is None:
            self.forward(ctx, xn, residual)
            return False
        h = self._hidden(ctx, xn)
        with kernels.phase("down"):
            kernels.linear_residual_norm(h, self.w_down, None, residual, args[0], args[1], out)
        return True


register_part("ffn", "swiglu", SwiGlu)
