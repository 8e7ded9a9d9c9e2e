"""Pre-norm residual arrangement: ``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/model.c:580-623)."""
from __future__ import annotations

from .base import Block, register_part


class PreNormResidual(Block):
    graph_safe = True

    def __init__(self, **_):
        pass

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache):
        xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
        norm1.forward(x, xn)
        mixer.forward(ctx, xn, x, cache, state, write_cache)
        norm2.forward(x, xn)
        ffn.forward(ctx, xn, x)


register_part("block", "prenorm_residual", PreNormResidual)
