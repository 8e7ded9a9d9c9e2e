"""RMSNorm: ``y_i = (x_i * rsqrt(mean(x^2) + eps)) * w_i`` (src/mathx.c:65-75, used at src/model.c:580, :611, :632)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Norm, register_part


class RmsNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, tensor: str, **_):
        self.size, self.eps, self.tensor = int(size), float(eps), tensor
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.tensor, (self.size,), init="norm")]

    def bind(self, tensors, run_dtype, device):
        self.weight = tensors[self.tensor].contiguous()

    def fused_args(self):
        return self.weight, self.eps

    def forward(self, x, out, rows=None):
        with kernels.phase("glue"):
            kernels.rmsnorm(x, self.weight, self.eps, out, rows)
        return out


register_part("norm", "rmsnorm", RmsNorm)
