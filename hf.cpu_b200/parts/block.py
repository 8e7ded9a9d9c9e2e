"""Pre-norm residual arrangement: ``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/model.c:580-623)."""
from __future__ import annotations

from .base import Block, register_part


class PreNormResidual(Block):
    graph_safe = True

    def __init__(self, **_):
        pass

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache, xn_ready=None, next_norm=None):
        if xn_ready is None:
            xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            norm1.forward(x, xn)
        else:
            xn = xn_ready
        xn2 = ctx.buf("block_xn2", x.shape, ctx.run_dtype)
        fused = getattr(mixer, "forward_then_norm", None)
        if not (fused and fused(ctx, xn, x, cache, state, write_cache, norm2, xn2)):
            if not fused:
                mixer.forward(ctx, xn, x, cache, state, write_cache)
            norm2.forward(x, xn2)
        fused = getattr(ffn, "forward_then_norm", None) if next_norm is not None else None
        if fused:
            nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            if not fused(ctx, xn2, x, next_norm, nxt):
                next_norm.forward(x, nxt)
            return nxt
        ffn.forward(ctx, xn2, x)
        return None


register_part("block", "prenorm_residual", PreNormResidual)
