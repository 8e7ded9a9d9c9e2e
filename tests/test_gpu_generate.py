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


def test_bfloat16_generation_follows_plain(tiny_folders):
    """Greedy generation in bfloat16 through the entry point gives the plain implementation's tokens (evaluated on the
    same bfloat16-stored weights) up to the first position where the plain logits hold a near-tie; sampled requests
    beside them run to their limit and are the same from run to run."""
    import hfcpu_b200
    folder = tiny_folders["B16"]
    prompts = list(make_requests("B", [19, 130, 64], seed=2).values())
    sess = hfcpu_b200.Session(folder, dtype="bfloat16", kv_block=8, kv_pages=128, max_seqs=4)
    out = sess.generate(prompts, temp=0, max_tokens=16)
    cfg, W = plain.read_folder(folder)
    exact = 0
    for p, comps in zip(prompts, out):
        got, want = comps[0].tokens, plain.greedy(cfg, W, p, 16)
        assert len(got) == 16 and comps[0].stop == "length"
        if got == want:
            exact += 1
            continue
        i = next(k for k in range(16) if got[k] != want[k])
        row = plain.forward(cfg, W, p + want[:i])[-1]
        gap = float(row[want[i]] - row[got[i]]) / float(row.abs().max())
        assert 0 <= gap < 3e-2, f"token {i}: plain prefers {want[i]} over {got[i]} by {gap:.3g} of the logits' range"
    assert exact >= 1
    a = sess.generate(prompts[:2], temp=0.7, seed=1, max_tokens=16, n=2)
    b = hfcpu_b200.Session(folder, dtype="bfloat16", kv_block=8, kv_pages=128, max_seqs=4).generate(
        prompts[:2], temp=0.7, seed=1, max_tokens=16, n=2)
    assert all(len(c.tokens) == 16 and c.stop == "length" for comps in a for c in comps)
    assert [[c.tokens for c in comps] for comps in a] == [[c.tokens for c in comps] for comps in b]


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


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("bfloat16", "B16")])
def test_running_ahead_of_the_host_changes_no_token(tiny_folders, dtype, name):
    """Steady decode steps are launched on the ids the sampling kernel has just written, before the host reads
    them.  The tokens must equal those of the step-by-step loop: greedy and sampled, requests of different
    lengths and limits, and an end token that arrives while the next step is already in flight."""
    import hfcpu_b200
    base = "A" if name == "A" else "B"
    prompts = list(make_requests(base, [5, 23, 40], seed=9).values())
    kw = dict(kv_block=BLOCK[base], kv_pages=96, max_seqs=4)
    for opts in (dict(temp=0, max_tokens=24), dict(temp=0.9, top_k=50, top_p=0.9, seed=3, max_tokens=21, n=2)):
        ahead_s = hfcpu_b200.Session(tiny_folders[name], dtype=dtype, **kw)
        ahead = ahead_s.generate(prompts, **opts)
        assert ahead_s.scheduler.stats["steps_ahead"] > 5
        plain_s = hfcpu_b200.Session(tiny_folders[name], dtype=dtype, **kw)
        plain_s.scheduler.run_ahead = False
        stepwise = plain_s.generate(prompts, **opts)
        assert plain_s.scheduler.stats["steps_ahead"] == 0
        assert [[c.tokens for c in comps] for comps in ahead] == [[c.tokens for c in comps] for comps in stepwise]
        assert ahead_s.engine.cache.pages_in_use() == 0
    # an end token in the middle: take a token the greedy run produced as the end token of a second run
    ref = hfcpu_b200.Session(tiny_folders[name], dtype=dtype, **kw).generate(prompts, temp=0, max_tokens=24)
    eos = ref[1][0].tokens[9]
    outs = []
    for ahead_on in (True, False):
        s = hfcpu_b200.Session(tiny_folders[name], dtype=dtype, eos_ids=[eos], **kw)
        s.scheduler.run_ahead = ahead_on
        outs.append(s.generate(prompts, temp=0, max_tokens=24))
        assert s.engine.cache.pages_in_use() == 0
        s.engine.cache.check()
    assert [[(c.tokens, c.stop) for c in comps] for comps in outs[0]] == [[(c.tokens, c.stop) for c in comps] for comps in outs[1]]
    assert outs[0][1][0].stop == "eos" and eos not in outs[0][1][0].tokens


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("float32", "B"), ("bfloat16", "A16"), ("bfloat16", "B16")])
def test_continuations_share_the_prompts_pages(tiny_folders, dtype, name):
    """Several completions of one prompt, and the next turn of a conversation: the tokens that are the same are
    computed once; in 32-bit every completion samples what it samples when it computes everything itself."""
    import hfcpu_b200
    folder = tiny_folders[name]
    name = name[:1]
    bs = BLOCK[name]
    prompt = make_requests(name, [150], seed=9)["r0"]
    kw = dict(temp=0.8, top_k=20, seed=3, max_tokens=12, n=3)
    outs = {}
    for share in (True, False):
        sess = hfcpu_b200.Session(folder, dtype=dtype, kv_block=bs, kv_pages=200, max_seqs=4, max_batched_tokens=64)
        sess.scheduler.share_prefixes = share
        outs[share] = [c.tokens for c in sess.generate(prompt, **kw)]
        st = sess.scheduler.stats
        assert st["tokens_shared"] == (2 * ((len(prompt) - 1) // bs * bs) if share else 0)
        assert sess.engine.cache.pages_in_use() == 0
        sess.engine.cache.check()
    if dtype == "float32":
        assert outs[True] == outs[False]
    # greedy: the three completions of a shared prompt are one and the same
    sess = hfcpu_b200.Session(folder, dtype=dtype, kv_block=bs, kv_pages=200, max_seqs=4, max_batched_tokens=64)
    same = [c.tokens for c in sess.generate(prompt, temp=0, max_tokens=10, n=3)]
    assert same[0] == same[1] == same[2]
    # the next turn starts on the pages kept of this one
    first = sess.generate(prompt, temp=0, max_tokens=10, keep_cache=True)[0].tokens
    assert first == same[0] and sess.scheduler.retained is not None
    follow = prompt + first + make_requests(name, [11], seed=10)["r0"]
    turn = sess.generate(follow, temp=0, max_tokens=6)[0].tokens
    rid = (sess._serial, 0, 0)
    # (where layers keep a window of keys only, the finished request has let go of pages that a query at the
    # start of the new tokens would still see: then nothing can be shared)
    windowed = any(g.spec.window for g in sess.engine.cache.groups)
    assert sess.scheduler.requests[rid].shared in ({0} if windowed else set()) | {(len(prompt) + len(first) - 1) // bs * bs}
    assert sess.scheduler.retained is None and sess.engine.cache.pages_in_use() == 0
    if dtype == "float32":
        cfg, W = plain.read_folder(folder)
        assert turn == plain.greedy(cfg, W, follow, 6)
    from hfcpu_b200 import kernels
    kernels.check_device_errors()
