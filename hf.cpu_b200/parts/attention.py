"""Grouped-query attention over the paged cache.

Per token: ``q, k, v = xn W{q,k,v}^T + b``; rotary on q and k; k (after rotation) and v go into
the cache at the token's slot; head h attends with the key/value head ``h // (H/G)`` over keys
``0 .. pos`` (or the last ``window`` of them), scores scaled by ``1/sqrt(head_dim)`` after the
dot, softmax, weighted values; ``out = att Wo^T`` is added to the residual
(src/model.c:581-609, :499-528).  q, k and v are one matrix product over concatenated rows
(src/model.c:581-585 runs the three jobs in one pass).
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.base import UnsupportedError
from ..weights.loader import TensorSpec, fused_rows
from .base import CacheSpec, Mixer, register_part


class PagedAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, out_bias: bool, window: int, position, prefix: str,
                 positions=None, names=None, **_):
        self.E, self.H, self.G, self.d = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        if self.H % self.G:
            raise UnsupportedError(f"unsupported attention geometry: {self.H} heads over {self.G} key/value heads")
        kernels.check_head_dim(self.d)
        self.qkv_bias, self.out_bias, self.window = bool(qkv_bias), bool(out_bias), int(window)
        self.rotary = (positions or {}).get(position) if position else None
        if position and self.rotary is None:
            raise UnsupportedError(f"attention names position encoding '{position}', which the plan does not define")
        n = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"}
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.scale = 1.0 / math.sqrt(self.d)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    @property
    def QD(self):
        return self.H * self.d

    @property
    def KD(self):
        return self.G * self.d

    def cache_spec(self):
        return CacheSpec(self.G, self.d, self.window)

    def step_arrays_key(self):
        return ("paged_attention_tiles", self.H // self.G)

    def step_arrays(self, batch):
        # the tile lists of the attention kernels: how they cut the step's tokens is the kernels' business
        return kernels.attention_step_arrays(batch.q_lens, self.H // self.G)

    def tensor_specs(self):
        s = [TensorSpec(self.names["q"] + ".weight", (self.QD, self.E)),
             TensorSpec(self.names["k"] + ".weight", (self.KD, self.E)),
             TensorSpec(self.names["v"] + ".weight", (self.KD, self.E)),
             TensorSpec(self.names["o"] + ".weight", (self.E, self.QD))]
        if self.qkv_bias:
            s += [TensorSpec(self.names[x] + ".bias", (n,)) for x, n in
                  (("q", self.QD), ("k", self.KD), ("v", self.KD))]
        if self.out_bias:
            s.append(TensorSpec(self.names["o"] + ".bias", (self.E,)))
        return s

    def bind(self, tensors, run_dtype, device):
        # q, k and v rows go straight into the one matrix the product reads, a tensor at a time
        self.w_qkv = fused_rows(tensors, [self.names[x] + ".weight" for x in "qkv"], device)
        if self.qkv_bias:
            self.b_qkv = fused_rows(tensors, [self.names[x] + ".bias" for x in "qkv"], device)
        self.w_o = tensors[self.names["o"] + ".weight"].contiguous()
        if self.out_bias:
            self.b_o = tensors[self.names["o"] + ".bias"].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.b_qkv, self.w_o, self.b_o)
                   if w is not None)

    def flops(self, q_lens, kv_lens):
        T = sum(q_lens)
        seen = 0                        # (query, key) pairs: token i of n new ones over a history of m sees m - n + i + 1
        for n, m in zip(q_lens, kv_lens):
            for_all = n * (m - n) + n * (n + 1) // 2
            if self.window > 0:
                for_all = sum(min(self.window, m - n + i + 1) for i in range(n)) if m > self.window else for_all
            seen += for_all
        return 2.0 * T * (self.w_qkv.numel() + self.w_o.numel()) + 4.0 * self.QD * seen

    def _attend(self, ctx, xn, cache, write_cache):
        T = xn.shape[0]
        qkv = ctx.buf("attn_qkv", (T, self.QD + 2 * self.KD), xn.dtype)
        q = ctx.buf("attn_q", (T, self.QD), xn.dtype)
        meta = ctx.group_meta(cache.group)
        cos_sin = self.rotary.cos_sin if self.rotary is not None else None
        n_rot = self.rotary.n_rot if self.rotary is not None else 0
        with kernels.phase("qkv"):
            kernels.linear_rope_kv(xn, self.w_qkv, self.b_qkv, qkv, cos_sin, n_rot, ctx.positions,
                                   meta.slots if write_cache else None, q, cache.k, cache.v, self.H, self.G, self.d)
        att = ctx.buf("attn_out", (T, self.QD), xn.dtype)
        with kernels.phase("attn"):
            kernels.paged_attention(q, cache.k, cache.v, meta, ctx, self.H, self.G, self.d,
                                    self.window, self.scale, att, tiles=ctx.arrays(self.step_arrays_key()))
        return att

    def forward(self, ctx, xn, residual, cache, state, write_cache):
        att = self._attend(ctx, xn, cache, write_cache)
        with kernels.phase("wo"):
            kernels.linear(att, self.w_o, self.b_o, residual, accumulate=True)

    def forward_then_norm(self, ctx, xn, residual, cache, state, write_cache, norm, out):
        args = norm.fused_args()
        if args is None:
            self.forward(ctx, xn, residual, cache, state, write_cache)
            return False
        att = self._attend(ctx, xn, cache, write_cache)
        with kernels.phase("wo"):
            kernels.linear_residual_norm(att, self.w_o, self.b_o, residual, args[0], args[1], out)
        return True


register_part("mixer", "paged_attention", PagedAttention)
