"""Generality of the parts: a toy mixer with state of its own, a feed-forward that routes tokens to experts, another
position encoding, a layer that runs twice, a layer that reads another layer's cache — all registered from here,
without a change to the framework's files.

Each case runs on the CPU with the torch stand-in for the kernels and, marked gpu, on the CUDA library.
"""
import dataclasses
from dataclasses import dataclass

import pytest
import torch

import plain_qwen2 as plain
import traces
from conftest import TINY_A, TINY_B, make_folder, make_requests

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]


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


# ---- a toy mixer with per-request state: a decaying sum of projected tokens ---------------------------
def _toy_parts():
    from hfcpu_b200.parts import Mixer, StateSpec
    from hfcpu_b200.weights import TensorSpec

    class DecayingSum(Mixer):
        """state_t = decay * state_{t-1} + x_t W^T;  out_t = state_t.  The state lives in the request's slot."""

        def __init__(self, hidden_size, decay, prefix, **_):
            self.E, self.decay, self.name = hidden_size, decay, f"{prefix}.w"
            self.w = None

        def state_spec(self):
            return StateSpec((self.E,), torch.float32)

        def tensor_specs(self):
            return [TensorSpec(self.name, (self.E, self.E))]

        def bind(self, tensors, run_dtype, device):
            self.w = tensors[self.name].float()

        def forward(self, ctx, xn, residual, cache, state, write_cache):
            assert cache is None and state is not None
            proj = xn.float() @ self.w.T
            for s in range(ctx.num_seqs):
                a, b, slot = ctx.h_cu_tokens[s], ctx.h_cu_tokens[s + 1], ctx.h_seq_slots[s]
                st = state[slot].clone()
                for t in range(a, b):                     # tokens of a request in order, from the slot's state
                    st = self.decay * st + proj[t]
                    residual[t] += st
                state[slot] = st
    return DecayingSum


@dataclass
class ToyConfig:
    """Alternates the toy mixer and paged attention; sizes unlike either tiny Qwen2 configuration."""
    architecture: str = "ToyForCausalLM"
    layers: int = 4
    hidden: int = 48
    heads: int = 3
    head_dim: int = 16
    ffn: int = 80
    vocab: int = 130
    positions: int = 256
    decay: float = 0.75

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: v for k, v in d.items() if k in {f.name for f in dataclasses.fields(cls)}})

    def to_dict(self):
        d = dataclasses.asdict(self)
        d["architectures"] = [d.pop("architecture")]
        return d

    def save(self, folder):
        import json, os
        os.makedirs(folder, exist_ok=True)
        json.dump(self.to_dict(), open(os.path.join(folder, "config.json"), "w"))

    # the architecture's side of a GGUF file: its metadata keys and its names for the tensors
    gguf_architecture = "toy"

    def gguf_metadata(self):
        return ([(f"toy.{k}", 4, getattr(self, k)) for k in ("layers", "hidden", "heads", "head_dim", "ffn", "positions")]
                + [("toy.decay", 6, self.decay)])

    def gguf_names(self):
        from hfcpu_b200.models import build_model_specs
        return {s.name: "t/" + s.name.replace("toy.", "").replace(".", "/") for s in build_model_specs(self)}

    def gguf_left_out(self):
        return []

    @classmethod
    def from_gguf(cls, meta, shapes, where=""):
        return cls(vocab=shapes["t/embed"][0], decay=round(meta["toy.decay"], 6),
                   **{k: meta[f"toy.{k}"] for k in ("layers", "hidden", "heads", "head_dim", "ffn", "positions")})

    def plan(self):
        from hfcpu_b200.config import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
        E = self.hidden
        norm = lambda n: PartSpec("rmsnorm", {"size": E, "eps": 1e-5, "tensor": n})
        layers = []
        for l in range(self.layers):
            p = f"toy.{l}"
            if l % 2 == 0:
                mixer = PartSpec("toy_decaying_sum", {"hidden_size": E, "decay": self.decay, "prefix": f"{p}.mix"})
            else:
                mixer = PartSpec("paged_attention", {"hidden_size": E, "num_heads": self.heads, "num_kv_heads": self.heads,
                                                     "head_dim": self.head_dim, "qkv_bias": False, "out_bias": False,
                                                     "window": 0, "position": "rope", "prefix": f"{p}.attn"})
            layers.append(LayerSpec(p, PartSpec("prenorm_residual"), norm(f"{p}.n1"), mixer, norm(f"{p}.n2"),
                                    PartSpec("swiglu", {"hidden_size": E, "intermediate_size": self.ffn, "prefix": f"{p}.ffn"})))
        return ModelPlan(E, self.vocab, self.positions,
                         PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "toy.embed"}),
                         {"rope": PartSpec("rotary", {"head_dim": self.head_dim, "n_rot": self.head_dim, "theta": 500.0})},
                         layers, [ScheduleEntry(l) for l in range(self.layers)], norm("toy.norm"),
                         PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "toy.head"}))


def _toy_reference(cfg, W, ids):
    """The toy model on one whole sequence, with the plain implementation's parts."""
    x = plain.embed(ids, W["toy.embed"])
    T = len(ids)
    cos, sin = plain.rope_angles(range(T), cfg.head_dim, 500.0, torch.float64)
    for l in range(cfg.layers):
        p = f"toy.{l}"
        xn = plain.rmsnorm(x, W[f"{p}.n1"], 1e-5)
        if l % 2 == 0:
            proj, st, outs = xn @ W[f"{p}.mix.w"].T, torch.zeros(cfg.hidden, dtype=torch.float64), []
            for t in range(T):
                st = cfg.decay * st + proj[t]
                outs.append(st)
            x = x + torch.stack(outs)
        else:
            H, d = cfg.heads, cfg.head_dim
            q = plain.rope((xn @ W[f"{p}.attn.q_proj.weight"].T).view(T, H, d), cos, sin, d)
            k = plain.rope((xn @ W[f"{p}.attn.k_proj.weight"].T).view(T, H, d), cos, sin, d)
            v = (xn @ W[f"{p}.attn.v_proj.weight"].T).view(T, H, d)
            x = x + plain.attention(q, k, v, H, H, 0).reshape(T, H * d) @ W[f"{p}.attn.o_proj.weight"].T
        xn = plain.rmsnorm(x, W[f"{p}.n2"], 1e-5)
        x = x + plain.swiglu_ffn(xn, W[f"{p}.ffn.gate_proj.weight"], W[f"{p}.ffn.up_proj.weight"], W[f"{p}.ffn.down_proj.weight"])
    return plain.rmsnorm(x, W["toy.norm"], 1e-5) @ W["toy.head"].T


@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_toy_mixer_with_state_is_registered_built_and_stepped(backend, tmp_path):
    import hfcpu_b200
    from hfcpu_b200.config import unregister_architecture
    from hfcpu_b200.parts import unregister_part
    hfcpu_b200.register_part("mixer", "toy_decaying_sum", _toy_parts())
    hfcpu_b200.register_architecture("ToyForCausalLM", ToyConfig)
    try:
        cfg = ToyConfig()
        folder = hfcpu_b200.write_random_model(cfg, str(tmp_path / "toy"), seed=4, dtype=torch.float32, std=0.3)
        model = hfcpu_b200.load_model(folder, torch.float32, backend)       # the class follows config.json
        assert type(model.config).__name__ == "ToyConfig"
        g = torch.Generator().manual_seed(0)
        reqs = {f"r{i}": torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for i, n in enumerate([40, 9, 77, 23])}
        _, W = plain.read_folder(folder)
        ref = {r: _toy_reference(cfg, W, ids) for r, ids in reqs.items()}
        for steps in (traces.whole(reqs), traces.portions(reqs), traces.mixed(reqs, max_live=3)):
            eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=traces.peak_tokens(steps), max_requests=3)
            assert sorted(eng.slots.tensors) == [0, 2] and eng.slots.bytes_per_request() == 2 * 48 * 4
            assert [g_.entries for g_ in eng.cache.groups] == [[1, 3]]
            got = traces.run_in_process(eng, steps, check=eng.cache.check)
            bad = traces.first_bad(got, ref, 1e-4)
            assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} ({bad[2]:.3g})"
            eng.slots.check()
    finally:
        unregister_part("mixer", "toy_decaying_sum")
        unregister_architecture("ToyForCausalLM")


def test_toy_architecture_brings_its_own_gguf_names(tmp_path, emu):
    """An architecture registered from outside exports to and loads from GGUF with metadata keys and tensor names of
    its own; the container code knows neither."""
    import hfcpu_b200
    from hfcpu_b200.config import unregister_architecture
    from hfcpu_b200.parts import unregister_part
    from hfcpu_b200.weights import load_tensors
    from hfcpu_b200.weights.gguf import GgufFile, write_gguf
    hfcpu_b200.register_part("mixer", "toy_decaying_sum", _toy_parts())
    hfcpu_b200.register_architecture("ToyForCausalLM", ToyConfig)
    hfcpu_b200.register_architecture("toy", ToyConfig)
    try:
        cfg = ToyConfig(layers=2, vocab=70)
        folder = hfcpu_b200.write_random_model(cfg, str(tmp_path / "toy"), seed=4, dtype=torch.float32, std=0.3)
        a = hfcpu_b200.load_model(folder, torch.float32, "cpu")
        path = str(tmp_path / "toy.gguf")
        write_gguf(path, cfg, load_tensors(folder, a.tensor_specs(), torch.float32, torch.device("cpu")))
        with GgufFile(path) as f:
            assert f.meta["general.architecture"] == "toy" and f.meta["toy.ffn"] == 80
            assert "t/1/attn/q_proj/weight" in f.names() and "t/0/mix/w" in f.names() and f.shape("t/embed") == (70, 48)
        b = hfcpu_b200.load_model(path, torch.float32, "cpu")
        assert dataclasses.replace(b.config, architecture=cfg.architecture) == cfg
        ids = [3, 9, 60, 2, 41]
        outs = []
        for m in (a, b):
            eng = hfcpu_b200.Engine(m, block_size=8, max_tokens=64, max_requests=1)
            eng.add_request("r")
            outs.append(eng.step([hfcpu_b200.StepEntry("r", ids, [4])]).clone())
        assert torch.equal(outs[0], outs[1])
    finally:
        unregister_part("mixer", "toy_decaying_sum")
        unregister_architecture("ToyForCausalLM")
        unregister_architecture("toy")


# ---- the run order is data: a layer named twice, a layer reading another entry's cache --------------------
def _scheduled_reference(cfg, W, ids, schedule):
    """schedule: list of (layer, cache_of); an entry with cache_of = j attends over the keys and values that
    entry j computed, with queries of its own."""
    H, G = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps, T = cfg["rms_norm_eps"], len(ids)
    W = {k: v.double() for k, v in W.items()}
    x = plain.embed(ids, W["model.embed_tokens.weight"])
    cos, sin = plain.rope_angles(range(T), d, cfg["rope_theta"], torch.float64)
    kv = {}
    for i, (l, cache_of) in enumerate(schedule):
        p = f"model.layers.{l}."
        xn = plain.rmsnorm(x, W[p + "input_layernorm.weight"], eps)
        q = plain.rope((xn @ W[p + "self_attn.q_proj.weight"].T + W[p + "self_attn.q_proj.bias"]).view(T, H, d), cos, sin, d)
        if cache_of is None:
            k = plain.rope((xn @ W[p + "self_attn.k_proj.weight"].T + W[p + "self_attn.k_proj.bias"]).view(T, G, d), cos, sin, d)
            v = (xn @ W[p + "self_attn.v_proj.weight"].T + W[p + "self_attn.v_proj.bias"]).view(T, G, d)
            kv[i] = (k, v)
        else:
            k, v = kv[cache_of]
        x = x + plain.attention(q, k, v, H, G, plain.window_of_layer(cfg, l)).reshape(T, H * d) @ W[p + "self_attn.o_proj.weight"].T
        xn = plain.rmsnorm(x, W[p + "post_attention_layernorm.weight"], eps)
        x = x + plain.swiglu_ffn(xn, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else W["lm_head.weight"]
    return plain.rmsnorm(x, W["model.norm.weight"], eps) @ head.T


@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_schedule_names_a_layer_twice_and_shares_a_cache(backend, tmp_path):
    import hfcpu_b200
    from hfcpu_b200.config import ScheduleEntry, config_from_dict
    folder = make_folder(dict(TINY_B, use_sliding_window=False), str(tmp_path / "m"), 5, torch.float32)
    cfg = config_from_dict(dict(TINY_B, use_sliding_window=False))
    order = [(0, None), (1, None), (1, None), (2, 1), (0, None)]
    plan = dataclasses.replace(cfg.plan(), schedule=[ScheduleEntry(l, c) for l, c in order])
    model = hfcpu_b200.Model(cfg, torch.float32, torch.device(backend), plan=plan)
    from hfcpu_b200.weights import load_tensors
    model.bind(load_tensors(folder, model.tensor_specs(), torch.float32, model.device))
    reqs = make_requests("B", [50, 21, 90], seed=12)
    pcfg, W = plain.read_folder(folder)
    ref = {r: _scheduled_reference(pcfg, W, ids, order) for r, ids in reqs.items()}
    for steps in (traces.whole(reqs), traces.mixed(reqs, max_live=2)):
        eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=traces.peak_tokens(steps), max_requests=2)
        assert [g.entries for g in eng.cache.groups] == [[0, 1, 2, 4]]           # entry 3 keeps no cache of its own
        got = traces.run_in_process(eng, steps, check=eng.cache.check)
        bad = traces.first_bad(got, ref, 1e-4)
        assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} ({bad[2]:.3g})"


# ---- a toy mixer with a paged cache and index arrays of its own for every step -------------------------------
def _toy_paged_mixer():
    from hfcpu_b200.parts import CacheSpec, Mixer
    from hfcpu_b200.weights import TensorSpec

    class CachedMean(Mixer):
        """v_t = x_t W^T goes into the paged cache; out_t = mean of v_0..v_t.  It cuts a step into tiles of three
        tokens (a tile shape no kernel of the framework has) and asks the engine for the tile list and for every
        token's cache slots as index arrays: the engine builds neither itself."""

        def __init__(self, hidden_size, prefix, **_):
            self.E, self.name, self.w = hidden_size, f"{prefix}.w", None

        def cache_spec(self):
            return CacheSpec(1, self.E, 0)

        def tensor_specs(self):
            return [TensorSpec(self.name, (self.E, self.E))]

        def bind(self, tensors, run_dtype, device):
            self.w = tensors[self.name].float()

        def step_arrays_key(self):
            return ("cached_mean_tiles", 3)

        def step_arrays(self, batch):
            seq, t0, nt, at = [], [], [], 0
            for s, n in enumerate(batch.q_lens):
                for a in range(0, n, 3):
                    seq.append(s), t0.append(at + a), nt.append(min(3, n - a))
                at += n
            return {"seq": seq, "t0": t0, "nt": nt, "first_pos": batch.starts}

        def forward(self, ctx, xn, residual, cache, state, write_cache):
            meta = ctx.group_meta(cache.group)
            arr = {k: v.tolist() for k, v in ctx.arrays(self.step_arrays_key()).items()}
            assert len(arr["first_pos"]) == ctx.num_seqs and sum(arr["nt"]) == ctx.num_tokens
            v = xn.float() @ self.w.T
            vf = cache.v.view(-1, self.E)
            vf[meta.slots.long()] = v.to(vf.dtype)
            table, bs = meta.block_table.tolist(), meta.block_size
            for s, t0, nt in zip(arr["seq"], arr["t0"], arr["nt"]):             # one tile of its own shape at a time
                for t in range(t0, t0 + nt):
                    pos = arr["first_pos"][s] + (t - ctx.h_cu_tokens[s])
                    slots = torch.tensor([table[s][j // bs] * bs + j % bs for j in range(pos + 1)], device=vf.device)
                    residual[t] += vf[slots].float().mean(0)
    return CachedMean


@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_toy_paged_mixer_brings_its_own_step_arrays(backend):
    import hfcpu_b200
    from hfcpu_b200.config import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
    from hfcpu_b200.parts import unregister_part
    from hfcpu_b200.weights import RandomSource
    hfcpu_b200.register_part("mixer", "toy_cached_mean", _toy_paged_mixer())
    try:
        E, V, L = 24, 50, 2
        norm = lambda n: PartSpec("rmsnorm", {"size": E, "eps": 1e-5, "tensor": n})
        layers = [LayerSpec(f"t.{l}", PartSpec("prenorm_residual"), norm(f"t.{l}.n1"),
                            PartSpec("toy_cached_mean", {"hidden_size": E, "prefix": f"t.{l}.mix"}), norm(f"t.{l}.n2"),
                            PartSpec("swiglu", {"hidden_size": E, "intermediate_size": 40, "prefix": f"t.{l}.ffn"}))
                  for l in range(L)]
        plan = ModelPlan(E, V, 128, PartSpec("embedding", {"vocab_size": V, "hidden_size": E, "tensor": "t.embed"}), {},
                         layers, [ScheduleEntry(l) for l in range(L)], norm("t.norm"),
                         PartSpec("linear_head", {"vocab_size": V, "hidden_size": E, "tensor": "t.head"}))
        model = hfcpu_b200.Model(None, torch.float32, torch.device(backend), plan=plan)
        src = RandomSource(model.tensor_specs(), 3, torch.float32, model.device, std=0.3)
        W = {n: src[n].double().cpu() for n in src.names()}
        model.bind(src)

        def reference(ids):
            x = plain.embed(ids, W["t.embed"])
            for l in range(L):
                v = plain.rmsnorm(x, W[f"t.{l}.n1"], 1e-5) @ W[f"t.{l}.mix.w"].T
                x = x + torch.cumsum(v, 0) / torch.arange(1, len(ids) + 1, dtype=torch.float64)[:, None]
                x = x + plain.swiglu_ffn(plain.rmsnorm(x, W[f"t.{l}.n2"], 1e-5), W[f"t.{l}.ffn.gate_proj.weight"],
                                         W[f"t.{l}.ffn.up_proj.weight"], W[f"t.{l}.ffn.down_proj.weight"])
            return plain.rmsnorm(x, W["t.norm"], 1e-5) @ W["t.head"].T
        g = torch.Generator().manual_seed(1)
        reqs = {f"r{i}": torch.randint(0, V, (n,), generator=g).tolist() for i, n in enumerate([37, 8, 50])}
        ref = {r: reference(ids) for r, ids in reqs.items()}
        for steps in (traces.whole(reqs), traces.portions(reqs), traces.mixed(reqs, max_live=2)):
            eng = hfcpu_b200.Engine(model, block_size=4, max_tokens=traces.peak_tokens(steps), max_requests=2)
            assert list(eng._array_owners) == [("cached_mean_tiles", 3)]
            got = traces.run_in_process(eng, steps, check=eng.cache.check)
            bad = traces.first_bad(got, ref, 1e-4)
            assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} ({bad[2]:.3g})"
    finally:
        unregister_part("mixer", "toy_cached_mean")


# ---- a feed-forward with routing and another position encoding, both defined here -------------------------
def _routed_ffn_part():
    from hfcpu_b200.parts import FeedForward
    from hfcpu_b200.weights import TensorSpec

    class Top1Experts(FeedForward):
        """Router logits in float32; the best expert's ``relu(x W1^T) W2^T`` weighted by its softmax share."""

        def __init__(self, hidden_size, inner, experts, prefix, **_):
            self.E, self.F, self.n, self.p = hidden_size, inner, experts, prefix
            self.router = self.w1 = self.w2 = None

        def tensor_specs(self):
            return [TensorSpec(f"{self.p}.router", (self.n, self.E)), TensorSpec(f"{self.p}.w1", (self.n, self.F, self.E)),
                    TensorSpec(f"{self.p}.w2", (self.n, self.E, self.F))]

        def bind(self, tensors, run_dtype, device):
            self.router, self.w1, self.w2 = (tensors[f"{self.p}.{k}"].float() for k in ("router", "w1", "w2"))

        def forward(self, ctx, xn, residual):
            x = xn.float()
            share = torch.softmax(x @ self.router.T, dim=-1)
            best = share.argmax(dim=-1)
            for e in range(self.n):
                rows = (best == e).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(x[rows] @ self.w1[e].T) @ self.w2[e].T
                    residual[rows] += y * share[rows, e:e + 1]
    return Top1Experts


def _scaled_rotary_part():
    from hfcpu_b200.parts import PositionEncoding

    class ScaledRotary(PositionEncoding):
        """Rotary angles of positions divided by ``factor``, over the first ``n_rot`` dimensions of a head only.
        The attention part takes any position part that offers ``cos_sin`` [positions, n_rot/2, 2] and ``n_rot``."""
        graph_safe = True

        def __init__(self, head_dim, n_rot, theta, factor, **_):
            self.head_dim, self.n_rot, self.theta, self.factor, self.cos_sin = head_dim, n_rot, theta, factor, None

        def prepare(self, max_positions, device):
            half = self.n_rot // 2
            inv = torch.tensor(self.theta, dtype=torch.float64) ** (-2.0 * torch.arange(half, dtype=torch.float64) / self.n_rot)
            ang = (torch.arange(max_positions, dtype=torch.float64) / self.factor)[:, None] * inv[None, :]
            self.cos_sin = torch.stack([ang.cos(), ang.sin()], dim=-1).float().contiguous().to(device)
    return ScaledRotary


@dataclass
class RoutedConfig:
    architecture: str = "RoutedToyForCausalLM"
    layers: int = 3
    hidden: int = 40
    heads: int = 5
    kv_heads: int = 1
    head_dim: int = 16
    n_rot: int = 8
    factor: float = 2.5
    inner: int = 24
    experts: int = 4
    vocab: int = 77
    positions: int = 256

    from_dict = classmethod(lambda cls, d: cls(**{k: v for k, v in d.items() if k in {f.name for f in dataclasses.fields(cls)}}))

    def to_dict(self):
        d = dataclasses.asdict(self)
        d["architectures"] = [d.pop("architecture")]
        return d

    def save(self, folder):
        import json, os
        os.makedirs(folder, exist_ok=True)
        json.dump(self.to_dict(), open(os.path.join(folder, "config.json"), "w"))

    def plan(self):
        from hfcpu_b200.config import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
        E = self.hidden
        norm = lambda n: PartSpec("rmsnorm", {"size": E, "eps": 1e-6, "tensor": n})
        layers = []
        for l in range(self.layers):
            p = f"rt.{l}"
            mixer = PartSpec("paged_attention", {"hidden_size": E, "num_heads": self.heads, "num_kv_heads": self.kv_heads,
                                                 "head_dim": self.head_dim, "qkv_bias": True, "out_bias": False,
                                                 "window": 0, "position": "scaled", "prefix": f"{p}.attn"})
            ffn = PartSpec("toy_top1_experts", {"hidden_size": E, "inner": self.inner, "experts": self.experts, "prefix": f"{p}.moe"})
            layers.append(LayerSpec(p, PartSpec("prenorm_residual"), norm(f"{p}.n1"), mixer, norm(f"{p}.n2"), ffn))
        return ModelPlan(E, self.vocab, self.positions,
                         PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "rt.embed"}),
                         {"scaled": PartSpec("toy_scaled_rotary", {"head_dim": self.head_dim, "n_rot": self.n_rot, "theta": 100.0,
                                                                   "factor": self.factor})},
                         layers, [ScheduleEntry(l) for l in range(self.layers)], norm("rt.norm"),
                         PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "rt.head"}))


def _routed_reference(cfg, W, ids):
    """The routed toy model on one whole sequence in float64.  Also returns the first position at which a router's
    two best experts are closer than a rounding error could decide (rows from there on are not compared)."""
    W = {k: v.double() for k, v in W.items()}
    x = plain.embed(ids, W["rt.embed"])
    T, H, G, d = len(ids), cfg.heads, cfg.kv_heads, cfg.head_dim
    half = cfg.n_rot // 2
    inv = torch.tensor(100.0, dtype=torch.float64) ** (-2.0 * torch.arange(half, dtype=torch.float64) / cfg.n_rot)
    ang = (torch.arange(T, dtype=torch.float64) / cfg.factor)[:, None] * inv[None, :]
    cos, sin = ang.cos(), ang.sin()
    unsure = T
    for l in range(cfg.layers):
        p = f"rt.{l}"
        xn = plain.rmsnorm(x, W[f"{p}.n1"], 1e-6)
        q = plain.rope((xn @ W[f"{p}.attn.q_proj.weight"].T + W[f"{p}.attn.q_proj.bias"]).view(T, H, d), cos, sin, cfg.n_rot)
        k = plain.rope((xn @ W[f"{p}.attn.k_proj.weight"].T + W[f"{p}.attn.k_proj.bias"]).view(T, G, d), cos, sin, cfg.n_rot)
        v = (xn @ W[f"{p}.attn.v_proj.weight"].T + W[f"{p}.attn.v_proj.bias"]).view(T, G, d)
        x = x + plain.attention(q, k, v, H, G, 0).reshape(T, H * d) @ W[f"{p}.attn.o_proj.weight"].T
        xn = plain.rmsnorm(x, W[f"{p}.n2"], 1e-6)
        share = torch.softmax(xn @ W[f"{p}.moe.router"].T, dim=-1)
        top = share.topk(2, dim=-1).values
        close = ((top[:, 0] - top[:, 1]) < 1e-4).nonzero().flatten()
        if close.numel():
            unsure = min(unsure, int(close[0]))
        best = share.argmax(dim=-1)
        y = torch.stack([torch.relu(xn[t] @ W[f"{p}.moe.w1"][best[t]].T) @ W[f"{p}.moe.w2"][best[t]].T * share[t, best[t]] for t in range(T)])
        x = x + y
    return plain.rmsnorm(x, W["rt.norm"], 1e-6) @ W["rt.head"].T, unsure


@pytest.mark.parametrize("backend", DEVICES, indirect=True)
def test_routed_feed_forward_and_another_position_encoding(backend, tmp_path):
    """A feed-forward that routes each token to one of four experts and a rotary encoding with scaled positions
    over half of each head, registered from here: the framework's attention, cache and step function run them
    unchanged, in every way of cutting the requests."""
    import hfcpu_b200
    from hfcpu_b200.config import unregister_architecture
    from hfcpu_b200.parts import unregister_part
    hfcpu_b200.register_part("ffn", "toy_top1_experts", _routed_ffn_part())
    hfcpu_b200.register_part("position", "toy_scaled_rotary", _scaled_rotary_part())
    hfcpu_b200.register_architecture("RoutedToyForCausalLM", RoutedConfig)
    try:
        cfg = RoutedConfig()
        folder = hfcpu_b200.write_random_model(cfg, str(tmp_path / "routed"), seed=9, dtype=torch.float32, std=0.3)
        model = hfcpu_b200.load_model(folder, torch.float32, backend)
        assert type(model.config).__name__ == "RoutedConfig"
        g = torch.Generator().manual_seed(1)
        reqs = {f"r{i}": torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for i, n in enumerate([33, 70, 12, 51])}
        _, W = plain.read_folder(folder)
        ref, sure = {}, {}
        for r, ids in reqs.items():
            ref[r], sure[r] = _routed_reference(cfg, W, ids)
        assert sum(sure.values()) > 0.8 * sum(len(v) for v in reqs.values()), "the routers are too often undecided to test anything"
        experts_used = set()
        for steps in (traces.whole(reqs), traces.portions(reqs), traces.mixed(reqs, max_live=3)):
            eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=traces.peak_tokens(steps), max_requests=3)
            got = traces.run_in_process(eng, steps, check=eng.cache.check)
            got = {(r, pos): row for (r, pos), row in got.items() if pos < sure[r]}
            assert len(got) > 50
            bad = traces.first_bad(got, ref, 1e-4)
            assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} ({bad[2]:.3g})"
    finally:
        unregister_part("ffn", "toy_top1_experts")
        unregister_part("position", "toy_scaled_rotary")
        unregister_architecture("RoutedToyForCausalLM")
