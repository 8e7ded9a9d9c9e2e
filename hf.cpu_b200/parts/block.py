"""Pre-norm residual arrangement: ``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/model.c:580-623)."""
from __future__ import annotations

from .base import Block, register_part


class PreNormResidual(Block):
    graph_safe = True

    def __init__(self, **_):
        pass

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache, xn_ready=None, next_norm=None,
                next_mixer=None):
        if xn_ready is None:
            xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            norm1.forward(x, xn)
        else:
            xn = xn_ready
        xn2 = ctx.buf("block_xn2", x.shape, ctx.run_dtype)
        import os
        pf = int(os.environ.get("HFB_PREFETCH_MB", "0"))
        if pf and ctx.num_tokens <= 128 and hasattr(ffn, "w_gate_up"):
            from .. import kernels
            b = kernels.backend()
            if hasattr(b, "prefetch_l2"):
                w = ffn.w_gate_up
                rows = min(w.shape[0], b.sm_count * 128)
                b.prefetch_l2(w, rows, (pf << 20) // rows)
        fused = getattr(mixer, "forward_then_norm", None)
        done = False
        if fused:
            # the row factor of norm2 may be left to the feed-forward's first product, if that part can apply it
            extra = {"defer": True} if getattr(ffn, "takes_row_scale", False) else {}
            done = fused(ctx, xn, x, cache, state, write_cache, norm2, xn2, **extra)
        else:
            mixer.forward(ctx, xn, x, cache, state, write_cache)
        if done is False or done is None:
            norm2.forward(x, xn2)
            done = True
        h_in = xn2 if done is True else done
        fused = getattr(ffn, "forward_then_norm", None) if next_norm is not None else None
        if fused:
            nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            extra = {"defer": True} if getattr(next_mixer, "takes_row_scale", False) else {}
            done = fused(ctx, h_in, x, next_norm, nxt, **extra)
            if done is False or done is None:
                next_norm.forward(x, nxt)
                done = True
            return nxt if done is True else done
        ffn.forward(ctx, h_in, x)
        return None


register_part("block", "prenorm_residual", PreNormResidual)
