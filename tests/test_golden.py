"""The plain implementation against what the reference's own C code computed (tests/golden/make_golden.py).

Greedy tokens must be identical; log-probabilities of the chosen token and of the top-5 candidates agree
within the bound the reference's own oracle uses for float weights (4e-3, tests/oracle.pl:18-23): the
reference keeps keys and values in float16 (src/model.c:599-600), the plain implementation in float64.
"""
import json
import os

import pytest
import torch

import plain_qwen2 as plain

HERE = os.path.dirname(os.path.abspath(__file__))


def _weights(record):
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors
    cfg = config_from_dict(record["config"])
    t = random_tensors(build_model_specs(cfg), record["seed"], torch.float32, std=record["std"])
    for k in t:
        if ".q_proj." in k or ".k_proj." in k:
            t[k] = t[k] * record["sharp"]
    return t


@pytest.mark.parametrize("name", ["A", "B", "A_rope8"])
def test_plain_matches_the_reference(name):
    record = json.load(open(os.path.join(HERE, "golden", f"tiny_{name}.json")))
    W = _weights(record)
    worst = 0.0
    for case in record["cases"]:
        ids = list(case["prompt"])
        for tok in case["tokens"]:
            logits = plain.forward(record["config"], W, ids)[-1]
            lp = torch.log_softmax(logits, dim=-1)
            assert int(torch.argmax(logits)) == tok["id"]
            worst = max(worst, abs(float(lp[tok["id"]]) - tok["logprob"]))
            # the same five candidates, except where the fifth and sixth are closer than the bound
            fifth = sorted((float(x) for x in lp), reverse=True)[4]
            assert all(float(lp[i]) >= fifth - 8e-3 for i, _ in tok["top"])
            worst = max(worst, max(abs(float(lp[i]) - v) for i, v in tok["top"]))
            ids.append(tok["id"])
    assert worst < 4e-3, worst


def test_gguf_round_trip(tmp_path):
    """The exporter writes what the importer (and the reference) reads: same names, shapes and values."""
    from hfcpu_b200.weights.gguf import GgufFile, read_gguf, write_gguf
    record = json.load(open(os.path.join(HERE, "golden", "tiny_B.json")))
    W = _weights(record)
    p = str(tmp_path / "m.gguf")
    write_gguf(p, record["config"], W)
    cfg, T = read_gguf(p)
    assert set(T) == set(W) and all(torch.equal(T[k], W[k]) for k in W)
    assert cfg.num_hidden_layers == 3 and cfg.head_dim == 32 and cfg.vocab_size == 1000 and cfg.rope_dim == 32
    assert not cfg.tie_word_embeddings and abs(cfg.rope_theta - 1e6) < 1 and cfg.num_key_value_heads == 3
    names = cfg.gguf_names()
    assert names["model.layers.2.self_attn.k_proj.bias"] == "blk.2.attn_k.bias"
    assert names["model.layers.1.mlp.down_proj.weight"] == "blk.1.ffn_down.weight" and len(names) == len(W)
    with GgufFile(p) as f:                                    # in the file: the reference's names, columns first
        assert set(f.names()) == set(names.values()) and f.meta["qwen2.rope.freq_base"] == 1e6
        assert f.shape("blk.0.ffn_up.weight") == (320, 192) and "qwen2.rope.dimension_count" not in f.meta
    from hfcpu_b200.weights import WeightFormatError
    data = open(p, "rb").read()
    for n in (0, 3, 20, 200, len(data) - 1):
        open(p, "wb").write(data[:n])
        with pytest.raises(WeightFormatError):
            read_gguf(p)


@pytest.mark.parametrize("name", ["A", "A_rope8"])
def test_engine_loads_gguf(tmp_path, emu, name):
    """The engine on a GGUF file gives the reference's greedy tokens; with ``rope.dimension_count`` below the head
    size (src/model.c:132-133) only that many dimensions of each head are turned."""
    import hfcpu_b200
    from hfcpu_b200.weights.gguf import GgufFile, write_gguf
    record = json.load(open(os.path.join(HERE, "golden", f"tiny_{name}.json")))
    W = _weights(record)
    p = str(tmp_path / "m.gguf")
    write_gguf(p, record["config"], W)
    with GgufFile(p) as f:
        assert f.meta.get("qwen2.rope.dimension_count") == record["config"].get("rope_dim")
    model = hfcpu_b200.load_model(p, torch.float32, "cpu")
    assert model.positions["rope"].n_rot == (record["config"].get("rope_dim") or 16)
    eng = hfcpu_b200.Engine(model, block_size=16, max_tokens=128, max_requests=2)
    case = record["cases"][1]
    eng.add_request("g")
    feed, out = list(case["prompt"]), []
    for _ in case["tokens"]:
        tok = int(torch.argmax(eng.step([hfcpu_b200.StepEntry("g", feed, [len(feed) - 1])])[0]))
        out.append(tok)
        feed = [tok]
    assert out == [t["id"] for t in case["tokens"]]


def test_gguf_metadata_that_cannot_be_honoured_is_refused(tmp_path):
    """A rotary width that is odd or wider than the head (src/model.c:141-144) and scaled rotary frequencies."""
    from hfcpu_b200.config import UnsupportedError, config_from_dict
    from hfcpu_b200.weights.gguf import F32, STRING, U32, GgufSource, write_gguf_file
    record = json.load(open(os.path.join(HERE, "golden", "tiny_A.json")))
    W = _weights(record)
    cfg = config_from_dict(record["config"])
    names = cfg.gguf_names()
    base = [("general.architecture", STRING, "qwen2")] + cfg.gguf_metadata()
    p = str(tmp_path / "m.gguf")
    for extra, what in (([("qwen2.rope.dimension_count", U32, 18)], "rope_dim 18"),
                        ([("qwen2.rope.dimension_count", U32, 7)], "rope_dim 7"),
                        ([("qwen2.rope.scaling.type", STRING, "yarn")], "scaled rotary"),
                        ([("qwen2.rope.scaling.factor", F32, 4.0)], "scaled rotary")):
        write_gguf_file(p, base + extra, ((names[n], W[n]) for n in W if n in names))
        with pytest.raises(UnsupportedError, match=what):
            GgufSource(p, torch.float32, torch.device("cpu"))
    write_gguf_file(p, [("general.architecture", STRING, "mamba")], [])
    with pytest.raises(UnsupportedError, match="architecture 'mamba' is not supported yet"):
        GgufSource(p, torch.float32, torch.device("cpu"))


# ---- the sampler, against the reference's own sampler (tests/golden/sampler.json) -----------------------------
def _sampler_record():
    return json.load(open(os.path.join(HERE, "golden", "sampler.json")))


def test_generators_give_the_references_draws():
    """xorshift64* seeded as src/sample.c:9-13, 24 bits per draw (src/sample.c:23): the first draws for five seeds
    are the numbers the reference's ``hfc_rng_uniform`` printed."""
    import numpy as np
    from hfcpu_b200.sampling import Rng
    for rec in _sampler_record()["rng"]:
        mine, plain_rng = Rng(rec["seed"]), plain.Rng(rec["seed"])
        for u in rec["uniforms"]:
            assert np.float32(mine.uniform()) == np.float32(u) == np.float32(plain_rng.uniform())


def test_samplers_pick_the_references_tokens():
    """Rows of synthetic logits, nine settings, twelve draws in a row from one generator: the plain sampler and the
    engine's host sampler pick the token ``hfc_sample`` picked (src/sample.c:66-116), every time."""
    from conftest import sampler_logits
    from hfcpu_b200.sampling import Rng, SamplingParams, sample_host
    L = sampler_logits()
    n = 0
    for rec in _sampler_record()["picks"]:
        row = L[rec["row"]]
        a, b = plain.Rng(rec["seed"]), Rng(rec["seed"])
        p = SamplingParams(temp=rec["temp"], top_k=min(rec["top_k"], 1 << 30), top_p=rec["top_p"], min_p=rec["min_p"])
        for want in rec["tokens"]:
            assert plain.sample(row, rec["temp"], rec["top_k"], rec["top_p"], rec["min_p"], a) == want, rec
            assert sample_host(row, p, b) == want, rec
            n += 1
    assert n == 54 * 12


@pytest.mark.parametrize("name", ["A", "B"])
def test_sampled_generation_follows_the_reference(name):
    """``hfcpu --temp .. --top-k .. --top-p .. --min-p .. --seed S --n N`` on the tiny models: feeding the reference's
    own tokens back (so that one difference does not change what follows), the plain logits and the plain sampler
    with seed S + i for sequence i (src/ops.c:819) pick the reference's token.  The reference's logits carry the
    rounding of its float16 cache, so a draw that lands within that noise of a boundary between two candidates may
    fall on the neighbour: a difference must be between neighbours in the candidate order, and at most 5 % differ."""
    record = json.load(open(os.path.join(HERE, "golden", f"tiny_{name}.json")))
    W = _weights(record)
    total = differ = 0
    for run in record["sampled"]:
        assert len(run["sequences"]) == run["n"]
        for i, seq in enumerate(run["sequences"]):
            rng = plain.Rng(run["seed"] + i)
            ids = list(run["prompt"])
            for tok in seq:
                logits = plain.forward(record["config"], W, ids)[-1].float().numpy()
                got = plain.sample(logits, run["temp"], run["top_k"], run["top_p"], run["min_p"], rng)
                total += 1
                if got != tok:
                    order = sorted(range(len(logits)), key=lambda j: (-logits[j], j))
                    assert abs(order.index(got) - order.index(tok)) == 1, (run, i, got, tok)
                    differ += 1
                ids.append(tok)
        if run["n"] > 1:
            assert len({tuple(s) for s in run["sequences"]}) == run["n"]          # seed + i: the sequences differ
    assert total == 5 * 24 and differ <= total // 20, (differ, total)
