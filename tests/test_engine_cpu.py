"""Host-side logic of the step function against the plain implementation, on the CPU.

The kernels are replaced by the torch stand-in (tests/emu_backend.py); what is under test is the
batch building, the block tables, page reuse and the parts' composition.
"""
import random

import pytest
import torch

import plain_qwen2 as plain
from conftest import BLOCK, TINY


def _engine(folder, name, max_tokens, dtype=torch.float32):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folder, dtype, "cpu")
    return hfcpu_b200.Engine(model, block_size=BLOCK[name], max_tokens=max_tokens, max_requests=4)


def _plain_logits(folder, ids):
    cfg, W = plain.read_folder(folder)
    return plain.forward(cfg, W, ids).float()


def _rel(a, b):
    return float((a - b).abs().max() / b.abs().max())


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt_matches_plain(tiny_folders, emu, name):
    from hfcpu_b200 import StepEntry
    g = torch.Generator().manual_seed(1)
    n = 150 if name == "B" else 70
    ids = torch.randint(0, TINY[name]["vocab_size"], (n,), generator=g).tolist()
    eng = _engine(tiny_folders[name], name, 256)
    eng.add_request("a")
    logits = eng.step([StepEntry("a", ids, list(range(n)))])
    ref = _plain_logits(tiny_folders[name], ids)
    assert _rel(logits, ref) < 1e-4
    eng.finish_request("a")
    eng.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_and_mixed_with_page_reuse(tiny_folders, emu, name):
    from hfcpu_b200 import StepEntry
    rnd = random.Random(5)
    V = TINY[name]["vocab_size"]
    reqs = {r: [rnd.randrange(V) for _ in range(n)] for r, n in (("a", 90), ("b", 33), ("c", 140), ("d", 64), ("e", 20))}
    ref = {r: _plain_logits(tiny_folders[name], ids) for r, ids in reqs.items()}
    eng = _engine(tiny_folders[name], name, 320)       # too few pages for all five at once
    order = list(reqs)
    live, done, fed = [], set(), {r: 0 for r in reqs}
    sizes = [32, 7, 16, 2, 5, 64, 1, 3]
    worst, step = 0.0, 0
    while len(done) < len(reqs):
        while len(live) < 3 and order:
            r = order.pop(0)
            eng.add_request(r)
            live.append(r)
        entries = []
        for r in live:
            if rnd.random() < 0.25 and len(live) > 1:
                continue                                 # a request may sit a step out
            n = min(sizes[(step + len(entries)) % len(sizes)], len(reqs[r]) - fed[r])
            entries.append(StepEntry(r, reqs[r][fed[r]:fed[r] + n], list(range(n))))
        step += 1
        if not entries:
            continue
        logits = eng.step(entries)
        o = 0
        for e in entries:
            n = len(e.tokens)
            worst = max(worst, _rel(logits[o:o + n], ref[e.req][fed[e.req]:fed[e.req] + n]))
            o += n
            fed[e.req] += n
            if fed[e.req] == len(reqs[e.req]):
                eng.finish_request(e.req)
                live.remove(e.req)
                done.add(e.req)
        eng.cache.check()
    assert worst < 1e-4
    assert eng.cache.pages_in_use() == 0
