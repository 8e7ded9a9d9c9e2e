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


@pytest.mark.parametrize("name", ["A", "B"])
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
    from hfcpu_b200.weights.gguf import read_gguf, to_checkpoint_name, to_gguf_name, write_gguf
    record = json.load(open(os.path.join(HERE, "golden", "tiny_B.json")))
    W = _weights(record)
    p = str(tmp_path / "m.gguf")
    write_gguf(p, record["config"], W)
    cfg, T = read_gguf(p)
    assert set(T) == set(W) and all(torch.equal(T[k], W[k]) for k in W)
    assert cfg["num_hidden_layers"] == 3 and cfg["head_dim"] == 32 and cfg["vocab_size"] == 1000
    assert not cfg["tie_word_embeddings"] and abs(cfg["rope_theta"] - 1e6) < 1 and cfg["num_key_value_heads"] == 3
    assert to_gguf_name("model.layers.2.self_attn.k_proj.bias") == "blk.2.attn_k.bias"
    assert to_checkpoint_name("blk.11.ffn_down.weight") == "model.layers.11.mlp.down_proj.weight"
    from hfcpu_b200.weights import WeightFormatError
    data = open(p, "rb").read()
    for n in (0, 3, 20, 200, len(data) - 1):
        open(p, "wb").write(data[:n])
        with pytest.raises(WeightFormatError):
            read_gguf(p)


def test_engine_loads_gguf(tmp_path, emu):
    import hfcpu_b200
    from hfcpu_b200.weights.gguf import write_gguf
    record = json.load(open(os.path.join(HERE, "golden", "tiny_A.json")))
    W = _weights(record)
    p = str(tmp_path / "m.gguf")
    write_gguf(p, record["config"], W)
    model = hfcpu_b200.load_model(p, torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=16, max_tokens=128, max_requests=2)
    case = record["cases"][1]
    eng.add_request("g")
    feed, out = list(case["prompt"]), []
    for _ in case["tokens"]:
        tok = int(torch.argmax(eng.step([hfcpu_b200.StepEntry("g", feed, [len(feed) - 1])])[0]))
        out.append(tok)
        feed = [tok]
    assert out == [t["id"] for t in case["tokens"]]
