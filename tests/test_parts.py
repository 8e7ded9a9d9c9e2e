"""Each part alone against the plain implementation's function for it: norm, position encoding, feed-forward, mixer,
block, embedding and head.  On the CPU with the torch stand-in for the kernels and, marked gpu, on the CUDA library,
in float32 and bfloat16, at sizes of their own (not a model configuration's)."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_qwen2 as plain

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.fixture
def backend(request):
    from hfcpu_b200 import kernels
    from emu_backend import EmuBackend
    dev = request.param
    old = kernels._backend
    if dev == "cpu":
        kernels.set_backend(EmuBackend())
    yield dev
    kernels.set_backend(old)


def rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max() / b.double().abs().max())


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return torch.randn(*shape, generator=g) * scale


class Ctx(SimpleNamespace):
    """The little of a step's context that a token-wise part needs: scratch buffers."""

    def buf(self, name, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_rmsnorm_part(backend, dtype):
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.parts import make_part
    E = 200
    norm = make_part("norm", PartSpec("rmsnorm", {"size": E, "eps": 3e-5, "tensor": "n.w"}))
    assert [(s.name, s.shape, s.init) for s in norm.tensor_specs()] == [("n.w", (E,), "norm")]
    w = (rnd(E) * 0.3 + 1).to(dtype)
    norm.bind({"n.w": w.to(backend)}, dtype, torch.device(backend))
    x = rnd(37, E, scale=2.0).to(backend)
    out = torch.empty(37, E, dtype=dtype, device=backend)
    norm.forward(x, out)
    assert rel(out, plain.rmsnorm(x.double().cpu(), w.double(), 3e-5)) < TOL[dtype]
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=backend)
    some = torch.empty(3, E, dtype=dtype, device=backend)
    norm.forward(x, some, rows=rows)
    assert torch.equal(some, out[rows.long()])
    assert norm.fused_args()[1] == 3e-5


def test_rotary_part_table():
    from hfcpu_b200.config import PartSpec, UnsupportedError
    from hfcpu_b200.parts import make_part
    rot = make_part("position", PartSpec("rotary", {"head_dim": 48, "n_rot": 32, "theta": 12345.0, "pairing": "half"}))
    rot.prepare(300, torch.device("cpu"))
    cos, sin = plain.rope_angles(range(300), 32, 12345.0, torch.float64)
    assert rot.cos_sin.shape == (300, 16, 2)
    assert float((rot.cos_sin[..., 0].double() - cos).abs().max()) < 1e-7
    assert float((rot.cos_sin[..., 1].double() - sin).abs().max()) < 1e-7
    with pytest.raises(UnsupportedError):
        make_part("position", PartSpec("rotary", {"head_dim": 48, "n_rot": 32, "theta": 1.0, "pairing": "interleaved"}))
    with pytest.raises(UnsupportedError):
        make_part("position", PartSpec("rotary", {"head_dim": 16, "n_rot": 32, "theta": 1.0}))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_swiglu_part(backend, dtype):
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.parts import make_part
    E, F, T = 72, 136, 19
    ffn = make_part("ffn", PartSpec("swiglu", {"hidden_size": E, "intermediate_size": F, "prefix": "f"}))
    assert sorted(s.name for s in ffn.tensor_specs()) == ["f.down_proj.weight", "f.gate_proj.weight", "f.up_proj.weight"]
    W = {"f.gate_proj.weight": rnd(F, E, scale=0.2, seed=1).to(dtype), "f.up_proj.weight": rnd(F, E, scale=0.2, seed=2).to(dtype),
         "f.down_proj.weight": rnd(E, F, scale=0.2, seed=3).to(dtype)}
    ffn.bind({k: v.to(backend) for k, v in W.items()}, dtype, torch.device(backend))
    xn = rnd(T, E).to(dtype)
    res = rnd(T, E, seed=9)
    want = res.double() + plain.swiglu_ffn(xn.double(), *(W[f"f.{n}_proj.weight"].double() for n in ("gate", "up", "down")))
    got = res.clone().to(backend)
    ffn.forward(Ctx(device=backend), xn.to(backend), got)
    assert rel(got, want) < TOL[dtype]
    # the same with the next norm applied in the product's tail
    norm = make_part("norm", PartSpec("rmsnorm", {"size": E, "eps": 1e-6, "tensor": "n.w"}))
    nw = (rnd(E) * 0.1 + 1).to(dtype)
    norm.bind({"n.w": nw.to(backend)}, dtype, torch.device(backend))
    got2, xn2 = res.clone().to(backend), torch.empty(T, E, dtype=dtype, device=backend)
    assert ffn.forward_then_norm(Ctx(device=backend), xn.to(backend), got2, norm, xn2) is True
    assert rel(got2, want) < TOL[dtype] and rel(xn2, plain.rmsnorm(want, nw.double(), 1e-6)) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_embedding_and_head_parts(backend, dtype):
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.parts import make_part
    V, E = 333, 40
    emb = make_part("embedding", PartSpec("embedding", {"vocab_size": V, "hidden_size": E, "tensor": "e"}))
    head = make_part("head", PartSpec("linear_head", {"vocab_size": V, "hidden_size": E, "tensor": "h", "tied_to": "e"}))
    table = rnd(V, E).to(dtype)
    tensors = {"e": table.to(backend)}
    for part in (emb, head):
        part.bind(tensors, dtype, torch.device(backend))
    ids = torch.tensor([0, 332, 7, 7, 100], dtype=torch.int32, device=backend)
    x = torch.empty(5, E, device=backend)
    emb.forward(ids, x)
    assert torch.equal(x.cpu(), plain.embed(ids.tolist(), table).float())
    xn = rnd(5, E, seed=4).to(dtype).to(backend)
    logits = torch.empty(5, V, device=backend)
    head.forward(xn, logits)
    assert rel(logits, xn.double().cpu() @ table.double().T) < TOL[dtype]
    assert head.weight is emb.table or head.weight.data_ptr() == emb.table.data_ptr()      # tied: the same memory


def _one_layer_engine(backend, dtype, window):
    """An engine around one layer of sizes of its own, to borrow a real step context and cache from."""
    import hfcpu_b200
    from hfcpu_b200.config import config_from_dict
    cfg = config_from_dict(dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=1, hidden_size=96, num_attention_heads=6,
                                num_key_value_heads=2, head_dim=32, intermediate_size=104, vocab_size=77,
                                max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=777.0, tie_word_embeddings=True,
                                use_sliding_window=window > 0, sliding_window=window, max_window_layers=0))
    model = hfcpu_b200.random_model(cfg, seed=8, dtype=dtype, device=backend, std=0.3)
    return cfg, model, hfcpu_b200.Engine(model, block_size=4, num_pages=40, max_requests=3)


@pytest.mark.parametrize("window", [0, 9])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_attention_mixer_and_block_parts(backend, dtype, window):
    """The mixer alone (projections, rotary, cache, attention, output projection into the residual), then the block
    around it, on two requests in one step, one of them continuing from an earlier portion."""
    from hfcpu_b200 import StepEntry
    cfg, model, eng = _one_layer_engine(backend, dtype, window)
    layer = model.layers[0]
    E, H, G, d = 96, 6, 2, 32
    g = torch.Generator().manual_seed(1)
    x_all = {r: torch.randn(n, E, generator=g) for r, n in (("a", 23), ("b", 14))}
    W = {n: t.double().cpu() for n, t in (("wqkv", layer.mixer.w_qkv), ("bqkv", layer.mixer.b_qkv), ("wo", layer.mixer.w_o))}
    n1, n2 = layer.norm1.weight.double().cpu(), layer.norm2.weight.double().cpu()

    def plain_mixer(x):
        T = x.shape[0]
        qkv = x.double() @ W["wqkv"].T + W["bqkv"]
        cos, sin = plain.rope_angles(range(T), d, 777.0, torch.float64)
        q = plain.rope(qkv[:, :H * d].reshape(T, H, d), cos, sin, d)
        k = plain.rope(qkv[:, H * d:(H + G) * d].reshape(T, G, d), cos, sin, d)
        v = qkv[:, (H + G) * d:].reshape(T, G, d)
        return plain.attention(q, k, v, H, G, window).reshape(T, H * d) @ W["wo"].T

    def plain_block(x):
        x = x.double()
        x = x + plain_mixer(plain.rmsnorm(x, n1, 1e-5))
        gu = layer.ffn.w_gate_up.double().cpu()
        return x + plain.swiglu_ffn(plain.rmsnorm(x, n2, 1e-5), gu[0::2], gu[1::2], layer.ffn.w_down.double().cpu())

    for what in ("mixer", "block"):
        for r in ("a", "b"):
            eng.add_request(r)
        fed = {"a": 0, "b": 0}
        for cut in ({"a": 10, "b": 14}, {"a": 13}):               # "a" comes in two portions, "b" whole beside the first
            entries = [StepEntry(r, [1] * n, []) for r, n in cut.items()]
            ctx = eng.prepare(entries)
            xs = torch.cat([x_all[r][fed[r]:fed[r] + n] for r, n in cut.items()])
            cache = ctx.entry_cache(0)
            if what == "mixer":
                res = torch.zeros(xs.shape[0], E, device=backend)
                layer.mixer.forward(ctx, xs.to(dtype).to(backend), res, cache, None, True)
                want = torch.cat([plain_mixer(x_all[r].to(dtype))[fed[r]:fed[r] + n] for r, n in cut.items()])
            else:
                res = xs.clone().to(backend)
                layer.block.forward(ctx, res, layer.norm1, layer.mixer, layer.norm2, layer.ffn, cache, None, True)
                want = torch.cat([plain_block(x_all[r])[fed[r]:fed[r] + n] for r, n in cut.items()])
            assert rel(res, want) < (TOL[dtype] if what == "mixer" else 2 * TOL[dtype]), (what, cut)
            for r, n in cut.items():
                eng.cache.advance(r, fed[r] + n)
                fed[r] += n
        for r in ("a", "b"):
            eng.finish_request(r)
    eng.cache.check()
