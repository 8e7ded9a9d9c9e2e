"""The plain implementation checked against closed forms and against itself."""
import math

import torch

import plain_qwen2 as plain
from conftest import TINY, make_requests


def test_rmsnorm_closed_form():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = plain.rmsnorm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0)
    r = 1 / math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 * r, 8 * r]], dtype=torch.float64))


def test_rope_rotates_pairs_half_apart_and_keeps_norms():
    d, T = 8, 5
    x = torch.randn(T, 2, d, dtype=torch.float64)
    cos, sin = plain.rope_angles(range(T), d, 10000.0, torch.float64)
    y = plain.rope(x, cos, sin, d)
    assert torch.allclose(y[0], x[0])                                       # position 0: no rotation
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    i, p = 1, 3
    th = p * 10000.0 ** (-2 * i / d)
    a, b = x[p, 0, i], x[p, 0, i + d // 2]
    assert abs(y[p, 0, i] - (a * math.cos(th) - b * math.sin(th))) < 1e-12
    assert abs(y[p, 0, i + d // 2] - (a * math.sin(th) + b * math.cos(th))) < 1e-12
    # dot products of rotated vectors depend on the distance of the positions only
    q = plain.rope(x[:1].expand(T, -1, -1), cos, sin, d)
    assert abs(float((q[1, 0] * q[3, 1]).sum() - (q[2, 0] * q[4, 1]).sum())) < 1e-12


def test_attention_is_causal_grouped_and_windowed():
    T, H, G, d = 12, 4, 2, 8
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (H, G, G))
    out = plain.attention(q, k, v, H, G, 0)
    k2, v2 = k.clone(), v.clone()
    k2[7:], v2[7:] = 0, 99
    assert torch.allclose(plain.attention(q, k2, v2, H, G, 0)[:7], out[:7])          # the future does not matter
    assert torch.allclose(out[0], v[0].repeat_interleave(H // G, dim=0))             # one key: its value
    v3 = v.clone()
    v3[:, 1] += 1                                                                    # heads 2, 3 read kv head 1
    d_out = plain.attention(q, k, v3, H, G, 0) - out
    assert float(d_out[:, :2].abs().max()) == 0 and torch.allclose(d_out[:, 2:], torch.ones_like(d_out[:, 2:]))
    w = plain.attention(q, k, v, H, G, 3)
    k4, v4 = k.clone(), v.clone()
    k4[:9], v4[:9] = 5, -7                                                           # position 11 sees keys 9, 10, 11
    assert torch.allclose(plain.attention(q, k4, v4, H, G, 3)[11], w[11])
    assert not torch.allclose(plain.attention(q, k4, v4, H, G, 4)[11], plain.attention(q, k, v, H, G, 4)[11])


def test_swiglu_formula():
    x = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    wg, wu, wd = torch.eye(2, dtype=torch.float64), 2 * torch.eye(2, dtype=torch.float64), torch.ones(1, 2, dtype=torch.float64)
    want = (1 / (1 + math.exp(-1))) * 2 + (-2 / (1 + math.exp(2))) * -4
    assert abs(float(plain.swiglu_ffn(x, wg, wu, wd)) - want) < 1e-12


def test_prefix_property_and_dtype_agreement(tiny_folders):
    """Logits at a position depend on the tokens up to it only; float32 and float64 evaluation agree."""
    for name in ("A", "B"):
        cfg, W = plain.read_folder(tiny_folders[name])
        ids = make_requests(name, [90], seed=4)["r0"]
        full = plain.forward(cfg, W, ids)
        assert torch.allclose(plain.forward(cfg, W, ids[:50]), full[:50], atol=1e-10)
        f32 = plain.forward(cfg, W, ids, torch.float32)
        assert float((f32.double() - full).abs().max() / full.abs().max()) < 2e-5
        assert full.shape == (90, TINY[name]["vocab_size"])


def test_window_changes_only_late_positions(tiny_folders):
    cfg, W = plain.read_folder(tiny_folders["B"])
    ids = make_requests("B", [100], seed=5)["r0"]
    windowed = plain.forward(cfg, W, ids)
    full = plain.forward(dict(cfg, use_sliding_window=False), W, ids)
    assert torch.allclose(windowed[:64], full[:64], atol=1e-10)       # up to 64 keys the window hides nothing
    assert float((windowed[64:] - full[64:]).abs().max()) > 1e-6
