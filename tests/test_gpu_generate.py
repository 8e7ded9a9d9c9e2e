"""Generation through the Python entry point and the command line, on the GPU."""
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen2 as plain
from conftest import BLOCK, ROOT, make_requests

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(tiny_folders, name):
    import hfcpu_b200
    folder = tiny_folders[name]
    sess = hfcpu_b200.Session(folder, dtype="float32", kv_block=BLOCK[name], kv_pages=64, max_seqs=4,
                              max_batched_tokens=48, batch=32)
    lengths = [7, 16, 33] if name == "A" else [1, 19, 64, 130]
    prompts = list(make_requests(name, lengths, seed=2).values())
    n_new = 8 if name == "A" else 16
    out = sess.generate(prompts, temp=0, max_tokens=n_new)
    cfg, W = plain.read_folder(folder)
    for p, comps in zip(prompts, out):
        assert comps[0].tokens == plain.greedy(cfg, W, p, n_new)
    assert sess.engine.cache.pages_in_use() == 0


def test_sampled_generation_survives_preemption(tiny_folders):
    import hfcpu_b200
    prompts = list(make_requests("A", [30, 30, 30], seed=6).values())
    kw = dict(temp=0.8, top_k=40, top_p=0.95, min_p=0.05, seed=5, max_tokens=40)
    roomy = hfcpu_b200.Session(tiny_folders["A"], dtype="float32", kv_pages=64, max_seqs=4).generate(prompts, **kw)
    tight_s = hfcpu_b200.Session(tiny_folders["A"], dtype="float32", kv_pages=11, max_seqs=4)
    tight = tight_s.generate(prompts, **kw)
    assert tight_s.scheduler.stats["preemptions"] > 0
    assert [c[0].tokens for c in roomy] == [c[0].tokens for c in tight]


def test_bfloat16_generation_runs(tiny_folders):
    import hfcpu_b200
    sess = hfcpu_b200.Session(tiny_folders["B16"], dtype="bfloat16", kv_block=8, kv_pages=128, max_seqs=4)
    prompts = list(make_requests("B", [19, 130], seed=2).values())
    out = sess.generate(prompts, temp=0.7, seed=1, max_tokens=16, n=2)
    assert all(len(c.tokens) == 16 and c.stop == "length" for comps in out for c in comps)


def test_command_line_generate(tiny_folders):
    prompt = make_requests("A", [12], seed=3)["r0"]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "hfb200"), "--stdin-mode", "none", "--op", "generate",
                        "--model", tiny_folders["A"], "--dtype", "fp32", "--kv-pages", "32", "--ctx-max", "256",
                        "--prompt-ids", " ".join(map(str, prompt)), "--temp", "0", "--max-tokens", "5"],
                       capture_output=True, timeout=300)
    assert r.returncode == 0, r.stderr.decode()
    toks = [int(l.split("id=")[1].split()[0]) for l in r.stdout.decode().splitlines() if l.startswith("@token")]
    cfg, W = plain.read_folder(tiny_folders["A"])
    assert toks == plain.greedy(cfg, W, prompt, 5)


def test_many_requests_under_pressure_match_plain(tiny_folders):
    """Twelve requests of mixed lengths through four slots, a small token budget and a pool too small for all of
    them: portions beside decodes, pages handed out again, preemption; every request's greedy tokens equal the plain
    implementation's."""
    import random
    import hfcpu_b200
    folder = tiny_folders["A"]
    rnd = random.Random(11)
    prompts = [[rnd.randrange(512) for _ in range(n)] for n in (90, 150, 40, 120, 17, 100, 3, 140, 60, 1, 130, 75)]
    sess = hfcpu_b200.Session(folder, dtype="float32", kv_block=16, kv_pages=20, max_seqs=4, max_batched_tokens=48, batch=32)
    out = sess.generate(prompts, temp=0, max_tokens=12)
    cfg, W = plain.read_folder(folder)
    for p, comps in zip(prompts, out):
        assert comps[0].stop == "length" and comps[0].tokens == plain.greedy(cfg, W, p, 12)
    st = sess.scheduler.stats
    assert st["preemptions"] > 0 and st["steps"] > 20
    sess.engine.cache.check()
    assert sess.engine.cache.pages_in_use() == 0 and sess.engine.slots.free_count == 4
