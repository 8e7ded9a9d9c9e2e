"""Token embedding (row gather into the float32 residual, src/model.c:566-571) and the output head
(final norm rows times the head matrix, float32 logits, src/model.c:629-637; tied head = the
embedding matrix, src/model.c:156-158)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part, register_part


class Embedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tensor: str, **_):
        self.vocab_size, self.hidden_size, self.tensor = int(vocab_size), int(hidden_size), tensor
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.tensor, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, run_dtype, device):
        self.table = tensors[self.tensor].contiguous()

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        with kernels.phase("embed"):
            kernels.embed(token_ids, self.table, out)
        return out


class LinearHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tensor: str, tied_to=None, **_):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tensor, self.tied_to = tensor, tied_to
        self.weight = None

    def tensor_specs(self):
        # a tied head reads the embedding; a checkpoint that carries a copy of the head anyway is accepted
        shape = (self.vocab_size, self.hidden_size)
        specs = [TensorSpec(self.tensor, shape, optional=bool(self.tied_to))]
        if self.tied_to:
            specs.append(TensorSpec(self.tied_to, shape))       # declared by both: the loader makes it once
        return specs

    def bind(self, tensors, run_dtype, device):
        self.weight = tensors[self.tied_to if self.tied_to else self.tensor].contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def flops(self, rows):
        return 2.0 * rows * self.weight.numel()

    def forward(self, xn: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        with kernels.phase("head"):
            kernels.linear(xn, self.weight, None, logits, accumulate=False)
        return logits


register_part("embedding", "embedding", Embedding)
register_part("head", "linear_head", LinearHead)
