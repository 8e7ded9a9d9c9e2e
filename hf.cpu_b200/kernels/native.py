"""ctypes binding of the CUDA library: the only kernel backend of the product.

Every method takes torch tensors on the GPU, checks what the C entry point cannot (devices,
contiguity), passes raw pointers and the current torch stream, and raises on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from . import build as _build

HFB_ENOTSUP = 2          # status of csrc/hfb200.h: not a case for this kernel, nothing was launched

_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)
if _raw_stream is None or _current_device is None:            # (another torch: the documented way)
    _raw_stream = lambda index: torch.cuda.current_stream(index).cuda_stream
    _current_device = torch.cuda.current_device


class KernelError(RuntimeError):
    pass


F32, BF16 = 0, 1


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _p(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


class NativeBackend:
    name = "native"

    def __init__(self):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: this engine has no CPU path")
        path = _build.build()
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the CUDA library {path} could not be loaded: {e}") from None
        self.lib.hfb_last_error.restype = ctypes.c_char_p
        self.lib.hfb_linear_tc_workspace.restype = ctypes.c_size_t
        self.lib.hfb_attention_fast_scratch.restype = ctypes.c_size_t
        # "fast": tiled tensor-core attention where the sizes allow; "plain": one block per (token, head) always
        self.attention = os.environ.get("HFB_ATTENTION", "fast")
        self.attention_tc = os.environ.get("HFB_ATTN_TC", "1") != "0"     # tcgen05 attention for prompt portions
        self.attention_tc2 = os.environ.get("HFB_ATTN_TC2", "1") != "0"   # its form with two query tiles per CTA
        # the two-tile form takes over once there is a work item for every SM this many times over (tests set 0)
        self.tc2_min_rounds = 0.55                # items per SM from which head size 128 takes the two-tile attention kernel
        self.decode_ctas_per_sm = 2               # CTAs of the decode attention kernel per SM, over all requests' splits
        self.decode_stages = 3                    # tiles of 64 keys in flight per CTA (measured again: 1 or 3 CTAs, 2 or 4 stages lose 0.4-7 %)
        self.sm_count = torch.cuda.get_device_properties(0).multi_processor_count
        # "tc": tensor-core products where the operands allow; "plain": the float32-accumulating SIMT kernel always
        self.gemm = os.environ.get("HFB_GEMM", "tc")
        self._ws = None
        self._argmax_ws = None
        # decode attention: the CTA that stores a tile's last split merges the splits (False: a second kernel does)
        self.merge_in_kernel = True
        self.rope_in_epilogue = os.environ.get("HFB_ROPE_EPILOGUE", "1") != "0"     # prompts: q|k|v product rotates and writes the cache
        self._counters = None
        self.lib.hfb_linear_tc_partials_workspace.restype = ctypes.c_size_t
        self.lib.hfb_argmax2_scratch.restype = ctypes.c_size_t
        self.path = path
        self.launches = 0          # kernels launched through this binding (one per successful call)

    def _stream(self):
        # the raw handle of torch's current stream on the current device; asked for at every launch (a few hundred
        # a step when steps run kernel by kernel), so by the two C calls behind torch.cuda.current_stream(), which
        # itself costs 14 us a call
        return c_void_p(_raw_stream(_current_device()))

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise KernelError(f"{what}: {self.lib.hfb_last_error().decode()} (status {rc})")
        self.launches += 1

    @staticmethod
    def _on_gpu(*ts):
        for t in ts:
            if t is not None and (not t.is_cuda or not t.is_contiguous()):
                raise KernelError("kernel arguments must be contiguous CUDA tensors")

    # ---- entry points -------------------------------------------------------------------------
    def embed(self, ids, table, out):
        self._on_gpu(ids, table, out)
        T, (V, E) = ids.shape[0], table.shape
        self._check(self.lib.hfb_embed(_p(ids), _p(table), c_int(_dt(table)), _p(out), c_int(T), c_int(V), c_int(E),
                                       self._stream()), "embed")

    def rmsnorm(self, x, w, eps, out, rows):
        self._on_gpu(x, w, out, rows)
        M, E = out.shape
        self._check(self.lib.hfb_rmsnorm(_p(x), _p(w), c_int(_dt(w)), c_float(eps), _p(out), c_int(_dt(out)), _p(rows),
                                         c_int(M), c_int(E), self._stream()), "rmsnorm")

    def linear(self, a, w, bias, out, accumulate):
        self._on_gpu(a, w, bias, out)
        M, K = a.shape
        N = w.shape[0]
        if (self.gemm == "tc" and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
                and (bias is None or bias.data_ptr() % 16 == 0)):
            need = self.lib.hfb_linear_tc_workspace(c_int(M), c_int(N), c_int(K))
            if need:
                self._workspace(a.device)
                if need > self._ws.numel():
                    need = 0                                        # runs unsplit
            self._check(self.lib.hfb_linear_tc(_p(a), _p(w), _p(bias), c_int(_dt(bias) if bias is not None else 0),
                                               _p(out), c_int(_dt(out)), c_int(1 if accumulate else 0), c_int(M),
                                               c_int(N), c_int(K), _p(self._ws if need else None),
                                               ctypes.c_size_t(self._ws.numel() if need else 0), self._stream()),
                        "linear_tc")
            return
        self._check(self.lib.hfb_linear_plain(_p(a), c_int(_dt(a)), _p(w), c_int(_dt(w)), _p(bias),
                                              c_int(_dt(bias) if bias is not None else 0), _p(out), c_int(_dt(out)),
                                              c_int(1 if accumulate else 0), c_int(M), c_int(N), c_int(K),
                                              self._stream()), "linear")

    def rope_kv_write(self, qkv, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        self._on_gpu(qkv, cos_sin, positions, slots, q_out, k_cache, v_cache)
        T = qkv.shape[0]
        cache_slots = k_cache.shape[0] * k_cache.shape[1]
        npos = cos_sin.shape[0] if cos_sin is not None else 0
        self._check(self.lib.hfb_rope_kv_write(_p(qkv), c_int(_dt(qkv)), _p(cos_sin), c_int(n_rot), c_int(npos),
                                               _p(positions), _p(slots), _p(q_out), _p(k_cache), _p(v_cache),
                                               c_int64(cache_slots), c_int(T), c_int(H), c_int(G), c_int(d),
                                               self._stream()), "rope_kv_write")

    def paged_attention(self, q, k_cache, v_cache, meta, ctx, H, G, d, window, scale, out, tile_arrays):
        self._on_gpu(q, k_cache, v_cache, meta.block_table, ctx.token_seq, ctx.positions, out)
        T = q.shape[0]
        if (self.attention == "fast" and tile_arrays and q.dtype == torch.bfloat16 and d in (64, 128)
                and 64 % meta.block_size == 0):
            decode = ctx.max_q_len == 1

            def tiles(ratio, height):
                """(seq, t0, nt, count) of the tile list of that height, or None when the step brought none."""
                h = str(height)
                if h + ".seq" not in tile_arrays and decode and height == 4 and 64 // ratio >= 1:
                    h = "1"                                   # one token a tile fits the wider kernel too
                seq = tile_arrays.get(h + ".seq")
                if seq is None:
                    return None
                return seq, tile_arrays[h + ".t0"], tile_arrays[h + ".nt"], seq.shape[0]
            if (not decode and self.attention_tc and meta.block_size >= 8 and 128 % meta.block_size == 0
                    and H // G <= 128):
                # two 128-row tiles per CTA once there are items for more than half of the SMs: it does more per key
                # fetched and overlaps softmax and products, but has half as many items to spread (28 heads over 4: 60
                # items 22.7 against 17.9 us, 116 items 32.3 against 37.9 us; 40 over 8: 88 items 23.0 against 26.7 us).
                # Head size 64 has this form only and always takes it (16 items: 14.6 us against 17.7 us of mma.sync)
                tiling = tiles(H // G, 16) if self.attention_tc2 else None
                enough = self.tc2_min_rounds * self.sm_count if d == 128 else 0
                if tiling is not None and tiling[3] * G >= enough:
                    tile_seq, tile_t0, tile_nt, n_tiles = tiling
                    self._check(self.lib.hfb_attention_tc2(
                        _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                        _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(meta.block_size),
                        c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out), c_int(T), c_int(H), c_int(G),
                        c_int(d), self._stream()), "attention_tc2")
                    return
                tiling = tiles(H // G, 8) if d == 128 else None      # tiles of 128 rows, as the 8-warp kernel's
                if tiling is not None:
                    tile_seq, tile_t0, tile_nt, n_tiles = tiling
                    self._check(self.lib.hfb_attention_tc(
                        _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                        _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(meta.block_size),
                        c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out), c_int(T), c_int(H), c_int(G),
                        c_int(d), self._stream()), "attention_tc")
                    return
            # single tokens: the decode kernel (16 rows a tile, keys and values by TMA) where the pages are at least 8
            # tokens; smaller pages take the 4-warp kernel with one token a tile
            decode_tma = decode and meta.block_size >= 8
            warps = 4
            tiling = tiles(H // G, 1 if decode_tma else warps)
            if tiling is None and not decode:
                warps = 8
                tiling = tiles(H // G, 8)
            if tiling is not None:
                tile_seq, tile_t0, tile_nt, n_tiles = tiling
                splits, stages = 1, 2
                if decode:
                    # about `decode_ctas_per_sm` CTAs per SM in all; with one per SM the deep pipeline fits
                    hint = getattr(ctx, "decode_split_hint", max(1, ((ctx.max_kv_len + 63) // 64) // 2))
                    splits = max(1, min(self.decode_ctas_per_sm * self.sm_count // max(1, n_tiles * G), hint))
                    stages = self.decode_stages
                else:
                    # short portions over a long context (the end of a prompt, a prompt behind a shared prefix): few
                    # tiles would each walk all the keys alone; their keys are split too, 256 to a CTA at least
                    splits = max(1, min(2 * self.sm_count // max(1, n_tiles * G), ((ctx.max_kv_len + 63) // 64) // 4, 64))
                need = self.lib.hfb_attention_fast_scratch(c_int(T), c_int(H), c_int(d), c_int(splits))
                scratch = ctx.buf("attn_scratch", (need,), torch.uint8) if need else None
                if decode_tma:
                    # the keys and values come by TMA, a warp of their own keeps them coming; the CTA that stores a
                    # tile's last split merges the splits (merge_in_kernel off: a second kernel does)
                    counters = None
                    if self.merge_in_kernel and splits > 1 and n_tiles * G <= 4096:
                        if self._counters is None or self._counters.device != q.device:
                            self._counters = torch.zeros(4096, dtype=torch.int32, device=q.device)
                        counters = self._counters
                    self._check(self.lib.hfb_attention_decode(
                        _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                        _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(stages), c_int(splits),
                        c_int(meta.block_size), c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out),
                        _p(scratch), ctypes.c_size_t(need), c_int(T), c_int(H), c_int(G), c_int(d), _p(counters),
                        c_int(counters.numel() if counters is not None else 0), self._stream()), "attention_decode")
                    if splits > 1 and counters is None:
                        self.launches += 1
                    return
                self._check(self.lib.hfb_attention_fast(
                    _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                    _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(warps), c_int(stages), c_int(splits),
                    c_int(meta.block_size), c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out),
                    _p(scratch), ctypes.c_size_t(need), c_int(T), c_int(H), c_int(G), c_int(d), self._stream()),
                    "attention_fast")
                if splits > 1:
                    self.launches += 1
                return
        self._check(self.lib.hfb_attention_plain(_p(q), _p(k_cache), _p(v_cache), c_int(_dt(q)), _p(meta.block_table),
                                                 c_int(meta.max_blocks), _p(ctx.token_seq), _p(ctx.positions),
                                                 c_int(meta.block_size), c_int64(k_cache.shape[0]), c_int(window),
                                                 c_float(scale), _p(out), c_int(T), c_int(H), c_int(G), c_int(d),
                                                 self._stream()), "attention")

    def swiglu(self, gu, out, interleaved):
        self._on_gpu(gu, out)
        T, F = out.shape
        self._check(self.lib.hfb_swiglu(_p(gu), _p(out), c_int(_dt(gu)), c_int(T), c_int(F), c_int(1 if interleaved else 0),
                                        self._stream()), "swiglu")

    def argmax(self, logits, out):
        self._on_gpu(logits, out)
        M, V = logits.shape
        need = self.lib.hfb_argmax2_scratch(c_int(M), c_int(V))
        if self._argmax_ws is None or self._argmax_ws.numel() < need:
            self._argmax_ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=logits.device)
        self._check(self.lib.hfb_argmax2(_p(logits), _p(out), c_int(M), c_int(V), _p(self._argmax_ws),
                                         ctypes.c_size_t(self._argmax_ws.numel()), self._stream()), "argmax")
        self.launches += 1

    # ---- fused forms: the tensor-core product with the next memory-bound step in its tail ------------------
    def _tc_ok(self, a, w, out=None):
        return (self.gemm == "tc" and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and (out is None or out.data_ptr() % 16 == 0))

    def _workspace(self, device):
        if self._ws is None or self._ws.device != device:
            self._ws = torch.empty(64 << 20, dtype=torch.uint8, device=device)     # split-K partials never need more
        return self._ws

    def _partials(self, a, w):
        """Split-K partial sums of a @ w.T in the workspace; returns (workspace, splits)."""
        M, K = a.shape
        N = w.shape[0]
        ws = self._workspace(a.device)
        need = self.lib.hfb_linear_tc_partials_workspace(c_int(M), c_int(N), c_int(K))
        if need == 0 or need > ws.numel():                      # 0: above 128 rows, and not a product that is split
            return None
        splits = c_int(0)
        self._check(self.lib.hfb_linear_tc_partials(_p(a), _p(w), c_int(M), c_int(N), c_int(K), _p(ws),
                                                    ctypes.c_size_t(ws.numel()), ctypes.byref(splits), self._stream()),
                    "linear_tc_partials")
        return ws, splits.value

    def linear_swiglu(self, a, w, gu_buf, out):
        self._on_gpu(a, w, out)
        M, K = a.shape
        N = w.shape[0]
        if self._tc_ok(a, w, out):
            self._check(self.lib.hfb_linear_tc_swiglu(_p(a), _p(w), _p(out), c_int(_dt(out)), c_int(M), c_int(N), c_int(K),
                                                      self._stream()), "linear_tc_swiglu")
            return
        self.linear(a, w, None, gu_buf, False)
        self.swiglu(gu_buf, out, True)

    def linear_residual_norm(self, a, w, bias, residual, norm_w, eps, xn_out):
        self._on_gpu(a, w, bias, residual, norm_w, xn_out)
        M, K = a.shape
        N = w.shape[0]
        part = self._partials(a, w) if self._tc_ok(a, w) else None
        if part is None:
            self.linear(a, w, bias, residual, True)
            if xn_out is not None:
                self.rmsnorm(residual, norm_w, eps, xn_out, None)
            return
        ws, splits = part
        self._check(self.lib.hfb_reduce_residual_norm(
            _p(ws), c_int(splits), c_int(M), c_int(N), _p(bias), c_int(_dt(bias) if bias is not None else 0), _p(residual),
            _p(norm_w), c_int(_dt(norm_w) if norm_w is not None else 0), c_float(eps), _p(xn_out),
            c_int(_dt(xn_out) if xn_out is not None else 0), self._stream()), "reduce_residual_norm")

    def linear_rope_kv(self, a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        self._on_gpu(a, w, bias, cos_sin, positions, slots, q_out, k_cache, v_cache)
        M, K = a.shape
        if (self.rope_in_epilogue and M >= 256 and self._tc_ok(a, w, q_out) and q_out.dtype == torch.bfloat16
                and k_cache.dtype == torch.bfloat16 and d in (64, 128) and n_rot == d and cos_sin is not None
                and (bias is None or (bias.dtype == torch.bfloat16 and bias.data_ptr() % 16 == 0))):
            # many tokens: rotation and the cache write run in the product's epilogue
            rc = self.lib.hfb_linear_tc_rope_kv(
                _p(a), _p(w), _p(bias), _p(cos_sin), c_int(cos_sin.shape[0]), _p(positions), _p(slots), _p(q_out),
                _p(k_cache), _p(v_cache), c_int64(k_cache.shape[0] * k_cache.shape[1]), c_int(M), c_int(K), c_int(H),
                c_int(G), c_int(d), self._stream())
            if rc != HFB_ENOTSUP:
                self._check(rc, "linear_tc_rope_kv")
                return
        part = self._partials(a, w) if self._tc_ok(a, w) else None
        if part is None:
            self.linear(a, w, bias, qkv_buf, False)
            self.rope_kv_write(qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d)
            return
        ws, splits = part
        cache_slots = k_cache.shape[0] * k_cache.shape[1]
        npos = cos_sin.shape[0] if cos_sin is not None else 0
        self._check(self.lib.hfb_reduce_rope_kv(
            _p(ws), c_int(splits), c_int(_dt(q_out)), _p(bias), c_int(_dt(bias) if bias is not None else 0), _p(cos_sin),
            c_int(n_rot), c_int(npos), _p(positions), _p(slots), _p(q_out), _p(k_cache), _p(v_cache), c_int64(cache_slots),
            c_int(M), c_int(H), c_int(G), c_int(d), self._stream()), "reduce_rope_kv")

    def sample(self, logits, temps, top_ks, top_ps, min_ps, uniforms, out):
        self._on_gpu(logits, temps, top_ks, top_ps, min_ps, uniforms, out)
        M, V = logits.shape
        self._check(self.lib.hfb_sample(_p(logits), c_int(M), c_int(V), _p(temps), _p(top_ks), _p(top_ps), _p(min_ps),
                                        _p(uniforms), _p(out), self._stream()), "sample")

    def error_word_async(self, host_word: torch.Tensor) -> None:
        """Queues a copy of the error word into ``host_word`` (pinned int32[1]); valid once the stream got there."""
        rc = self.lib.hfb_error_word_peek_async(c_void_p(host_word.data_ptr()), self._stream())
        if rc != 0:
            raise KernelError(f"error word: {self.lib.hfb_last_error().decode()} (status {rc})")

    def error_word(self) -> int:
        w = ctypes.c_int32(0)
        self._check(self.lib.hfb_error_word_take(ctypes.byref(w), self._stream()), "error word")
        if w.value and self._counters is not None:
            self._counters.zero_()             # a kernel that gave up may have left tile counts behind
        return w.value
