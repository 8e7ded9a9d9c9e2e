"""A plain, slow implementation of the Qwen2 dense decoder: whole sequences, no cache.

One function per part, written from the reference's formulas (file:line of ebowh/hf.cpu cited at
each function) and sharing no code with the engine.  It reads ``config.json`` as a plain dict and
the checkpoint tensors by name, and returns logits for every position of one token sequence.
The sliding window is not in the reference (its key loop always runs 0..pos, src/model.c:514); it
follows config.json's meaning as the benchmark configurations state it: layers with index >=
``max_window_layers`` see only keys j with 0 <= pos - j < ``sliding_window``.

Cross-checked once against the reference's own C model code on a tiny random model: see
tests/golden/make_golden.py.
"""
import json
import math
import os
import struct

import numpy as np
import torch


# ---- reading a model folder without the engine's loader -------------------------------------------
def read_folder(folder, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        raw = torch.from_numpy(np.frombuffer(data[b:en], dtype=np.uint8).copy())
        tensors[name] = raw.view(kinds[e["dtype"]]).reshape(e["shape"]).to(dtype)
    return cfg, tensors


# ---- parts -------------------------------------------------------------------------------------
def embed(ids, table):
    """x[t, :] = row id[t] of the embedding table (src/model.c:566-571)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)]


def rmsnorm(x, w, eps):
    """ss = sum x_i^2; r = 1/sqrt(ss/E + eps); y_i = (x_i * r) * w_i (src/mathx.c:65-75)."""
    mean = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return (x * (1.0 / torch.sqrt(mean + eps))) * w


def rope_angles(positions, n_rot, base, dtype):
    """theta_i(pos) = pos * base^(-2i/n_rot), i < n_rot/2 (src/model.c:468-477; the reference steps a
    float recurrence theta *= base^(-2/n_rot); the closed form is tools/ref-forward.pl:92-104)."""
    i = torch.arange(n_rot // 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / n_rot)
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def rope(x, cos, sin, n_rot):
    """Half-split pairing: (a, b) = (x[i], x[i + n_rot/2]); a' = a c - b s; b' = a s + b c; dimensions
    >= n_rot unchanged (src/model.c:479-493 with rope_neox, src/model.c:140).  x: [T, heads, d]."""
    half = n_rot // 2
    a, b = x[..., :half], x[..., half:n_rot]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, a * s + b * c, x[..., n_rot:]], dim=-1)


def attention(q, k, v, n_heads, n_kv_heads, window):
    """Head h uses key/value head h // (H/G); scores = (q . k) * (1/sqrt(d)) with the scale after the
    dot; causal: token t sees keys 0..t (src/model.c:499-520); softmax with the maximum subtracted
    (src/mathx.c:77-86); out = sum_j p_j v_j (src/model.c:522-526).  q: [T, H, d]; k, v: [T, G, d]."""
    T, H, d = q.shape
    rep = n_heads // n_kv_heads
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible = visible & (pos[:, None] - pos[None, :] < window)
    for h in range(H):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu_ffn(x, wg, wu, wd):
    """g = x Wg^T; u = x Wu^T; h = g / (1 + exp(-g)) * u; out = h Wd^T (src/model.c:612-623, src/mathx.c:34)."""
    g, u = x @ wg.T, x @ wu.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ wd.T


def window_of_layer(cfg, l):
    if cfg.get("use_sliding_window") and l >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return int(cfg["sliding_window"])
    return 0


def layer(x, cfg, W, l, cos, sin):
    """Pre-norm block: x += Wo attention(rope(q), rope(k), v); x += ffn(norm(x)) (src/model.c:580-623)."""
    H = cfg["num_attention_heads"]
    G = cfg.get("num_key_value_heads", H)
    d = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps = cfg.get("rms_norm_eps", 1e-5)
    p = f"model.layers.{l}."
    T = x.shape[0]
    xn = rmsnorm(x, W[p + "input_layernorm.weight"], eps)
    q = xn @ W[p + "self_attn.q_proj.weight"].T + W[p + "self_attn.q_proj.bias"]
    k = xn @ W[p + "self_attn.k_proj.weight"].T + W[p + "self_attn.k_proj.bias"]
    v = xn @ W[p + "self_attn.v_proj.weight"].T + W[p + "self_attn.v_proj.bias"]
    n_rot = cfg.get("rope_dim") or d          # the reference's rope.dimension_count (src/model.c:132-133)
    q = rope(q.view(T, H, d), cos, sin, n_rot)
    k = rope(k.view(T, G, d), cos, sin, n_rot)
    att = attention(q, k, v.view(T, G, d), H, G, window_of_layer(cfg, l)).reshape(T, H * d)
    x = x + att @ W[p + "self_attn.o_proj.weight"].T
    xn = rmsnorm(x, W[p + "post_attention_layernorm.weight"], eps)
    return x + swiglu_ffn(xn, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])


def forward(cfg, W, ids, dtype=torch.float64):
    """Logits [T, V] for every position of ``ids`` (src/model.c:545-640; head tied to the embedding when
    the checkpoint has no head matrix, src/model.c:156-158)."""
    W = {k: v.to(dtype) for k, v in W.items()}
    H = cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // H
    x = embed(ids, W["model.embed_tokens.weight"])
    cos, sin = rope_angles(range(len(ids)), cfg.get("rope_dim") or d, cfg.get("rope_theta", 10000.0), dtype)
    cos, sin = cos.to(x.device), sin.to(x.device)
    for l in range(cfg["num_hidden_layers"]):
        x = layer(x, cfg, W, l, cos, sin)
    xn = rmsnorm(x, W["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else W["lm_head.weight"]
    return xn @ head.T


def greedy(cfg, W, ids, n, dtype=torch.float64):
    """Greedy continuation: the first index of the maximum each time (src/sample.c:72-77)."""
    ids = list(ids)
    out = []
    for _ in range(n):
        logits = forward(cfg, W, ids, dtype)[-1]
        tok = int(torch.argmax(logits))        # torch.argmax returns the first maximum
        out.append(tok)
        ids.append(tok)
    return out


# ---- sampling (src/sample.c) -------------------------------------------------------------------
class Rng:
    """xorshift64* (src/sample.c:9-23)."""
    M = (1 << 64) - 1

    def __init__(self, seed):
        self.s = (seed * 0x9E3779B97F4A7C15 + 0x1234567) & self.M
        if self.s == 0:
            self.s = 0x2545F4914F6CDD1D

    def uniform(self):
        x = self.s
        x ^= x >> 12
        x ^= (x << 25) & self.M
        x ^= x >> 27
        self.s = x
        return np.float32(((x * 0x2545F4914F6CDD1D) & self.M) >> 40) / np.float32(16777216.0)


def sample(logits, temp, top_k, top_p, min_p, rng):
    """Greedy for temp <= 0; else top-k (ties: lower id first), softmax of (l - max)/temp, min-p, top-p,
    draw r = u * sum over the kept list, all in float32 (src/sample.c:66-116)."""
    l = np.asarray(logits, dtype=np.float32)
    if temp <= 0:
        return int(np.argmax(l))
    order = sorted(range(len(l)), key=lambda i: (-l[i], i))
    if 0 < top_k < len(l):
        order = order[:top_k]
    p = np.exp(((l[order] - l[order[0]]) / np.float32(temp)).astype(np.float32)).astype(np.float32)
    s = np.float32(0)
    for v in p:
        s = np.float32(s + v)
    p = (p / s).astype(np.float32)
    kept = len(p)
    if min_p > 0:
        kept = 0
        while kept < len(p) and p[kept] >= np.float32(min_p) * p[0]:
            kept += 1
        kept = max(kept, 1)
    if 0 < top_p < 1:
        cum = np.float32(0)
        for i in range(kept):
            cum = np.float32(cum + p[i])
            if cum >= np.float32(top_p):
                kept = i + 1
                break
    s = np.float32(0)
    for i in range(kept):
        s = np.float32(s + p[i])
    r = np.float32(rng.uniform() * s)
    cum = np.float32(0)
    for i in range(kept):
        cum = np.float32(cum + p[i])
        if r < cum:
            return int(order[i])
    return int(order[kept - 1])
