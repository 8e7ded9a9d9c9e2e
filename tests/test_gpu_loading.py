"""Loading on the GPU: shards, the staging path, what the device holds at its peak; and the workload of the 0.5B
benchmark configuration scaled to a test (many requests, chunked prompts beside decodes, a pool that forces preemption)."""
import json
import os
import random

import pytest
import torch

from conftest import TINY_C, make_requests

pytestmark = pytest.mark.gpu


def _shard(folder, n_shards, with_index):
    """Rewrites a single-file model folder as ``n_shards`` files named like a published checkpoint's."""
    from hfcpu_b200.weights import SafetensorsFile, weights_path, write_safetensors
    with SafetensorsFile(weights_path(folder)) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    os.remove(weights_path(folder))
    names, wmap = sorted(tensors), {}
    for i in range(n_shards):
        fn = f"model-{i + 1:05d}-of-{n_shards:05d}.safetensors"
        write_safetensors(os.path.join(folder, fn), {n: tensors[n] for n in names[i::n_shards]})
        wmap.update({n: fn for n in names[i::n_shards]})
    if with_index:
        json.dump({"metadata": {}, "weight_map": wmap}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_sharded_and_single_file_folders_give_the_same_logits(tmp_path, dtype):
    import hfcpu_b200
    from hfcpu_b200.config import config_from_dict
    dt = getattr(torch, dtype)
    ids = make_requests("C", [150], seed=5)["r0"]
    outs = []
    for kind in ("single", "index", "bare"):
        folder = hfcpu_b200.write_random_model(config_from_dict(TINY_C), str(tmp_path / kind), seed=6, dtype=torch.bfloat16, std=0.05)
        if kind != "single":
            _shard(folder, 3, kind == "index")
        model = hfcpu_b200.load_model(folder, dt, "cuda:0")
        assert len(model.files) == (1 if kind == "single" else 3)
        eng = hfcpu_b200.Engine(model, block_size=16, max_tokens=256, max_requests=1)
        eng.add_request("r")
        rows = [eng.step([hfcpu_b200.StepEntry("r", ids, [0, 77, 149])]).clone()]
        rows.append(eng.step([hfcpu_b200.StepEntry("r", [5], [0])]).clone())
        outs.append(torch.cat(rows))
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_loading_holds_little_more_than_the_weights(tmp_path):
    """Two layers at the 7B widths (vocabulary cut to 8,192 so that the file stays near 1 GB): while loading, the
    device never holds more than the weights bound so far and the one tensor in transit."""
    import hfcpu_b200
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import RandomSource, weights_path, write_safetensors
    cfg = config_from_dict(dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=3584,
                                num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, vocab_size=8192,
                                max_position_embeddings=4096, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False))
    folder = str(tmp_path / "wide")
    cfg.save(folder)
    write_safetensors(weights_path(folder), RandomSource(build_model_specs(cfg), 2, torch.bfloat16, torch.device("cuda:0")))
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    model = hfcpu_b200.load_model(folder, torch.bfloat16, "cuda:0")
    torch.cuda.synchronize()
    weights = sum(p.weight_bytes() for p in model.all_parts()) + model.embedding.table.numel() * 2
    tables = sum(p.cos_sin.numel() * 4 for p in model.positions.values())
    peak = torch.cuda.max_memory_allocated() - base
    assert peak <= 1.1 * weights + tables, (peak, weights)
    assert torch.cuda.memory_allocated() - base <= 1.01 * weights + tables
    # what was loaded is what was written: one tensor of the fused buffers against the source
    src = RandomSource(build_model_specs(cfg), 2, torch.bfloat16, torch.device("cuda:0"))
    g, u = src["model.layers.1.mlp.gate_proj.weight"], src["model.layers.1.mlp.up_proj.weight"]
    assert torch.equal(model.layers[1].ffn.w_gate_up[0::2], g) and torch.equal(model.layers[1].ffn.w_gate_up[1::2], u)


def test_many_requests_chunked_prompts_beside_decodes_at_half_b_widths(tmp_path):
    """32 requests with prompts of 1 to 1,024 tokens on two layers at the Qwen2.5-0.5B widths, prompts in portions of 256
    beside the decodes of others, a pool small enough to preempt: greedy tokens of the bfloat16 path equal the true
    32-bit path's up to the first token where the 32-bit logits hold a near-tie; sampled requests (temperature 0.7)
    run to their end beside them."""
    import hfcpu_b200
    from hfcpu_b200.config import config_from_dict
    cfg = config_from_dict(dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=896,
                                num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864, vocab_size=151936,
                                max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True))
    folder = hfcpu_b200.write_random_model(cfg, str(tmp_path / "half_b"), seed=8, dtype=torch.bfloat16, std=0.02)
    rnd = random.Random(3)
    prompts = [[rnd.randrange(cfg.vocab_size) for _ in range(rnd.randint(1, 1024))] for _ in range(32)]
    n_new = 24
    results = {}
    for dtype in ("float32", "bfloat16"):
        sess = hfcpu_b200.Session(folder, dtype=dtype, kv_block=16, kv_pages=260, max_seqs=8, max_batched_tokens=256 + 8,
                                  batch=256, ctx_max=2048)
        results[dtype] = sess.generate(prompts, temp=0, max_tokens=n_new)
        st = sess.scheduler.stats
        assert st["preemptions"] > 0, "the pool was meant to be too small for eight long requests"
        assert sess.engine.cache.pages_in_use() == 0
        sess.engine.cache.check()
        if dtype == "bfloat16":
            sampled = sess.generate(prompts[:8], temp=0.7, seed=3, max_tokens=n_new)
            assert all(c[0].stop == "length" and len(c[0].tokens) == n_new for c in sampled)
        else:
            engine32 = sess.engine
    same = near = 0
    for p, a, b in zip(prompts, results["float32"], results["bfloat16"]):
        ta, tb = a[0].tokens, b[0].tokens
        assert len(ta) == len(tb) == n_new
        if ta == tb:
            same += 1
            continue
        i = next(k for k in range(n_new) if ta[k] != tb[k])
        engine32.add_request("probe")
        ids = p + ta[:i]
        row = None
        for s in range(0, len(ids), 512):
            part = ids[s:s + 512]
            row = engine32.step([hfcpu_b200.StepEntry("probe", part, [len(part) - 1] if s + 512 >= len(ids) else [])])
        row = row[0]
        engine32.finish_request("probe")
        gap = float(row[ta[i]] - row[tb[i]]) / float(row.abs().max())
        assert 0 <= gap < 3e-2, f"token {i}: the 32-bit logits prefer {ta[i]} over {tb[i]} by {gap:.3g} of their range"
        near += 1
    assert same + near == 32 and same >= 8, (same, near)
