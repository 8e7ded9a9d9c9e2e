"""The scheduler's decisions, on the CPU (kernels replaced by the torch stand-in)."""
import pytest
import torch

import plain_qwen2 as plain
from conftest import BLOCK, TINY, make_requests


def _session(folder, name, pages, max_seqs=4, budget=64, chunk=0):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folder, torch.float32, "cpu")
    return hfcpu_b200.Session(model, kv_block=BLOCK[name], kv_pages=pages, max_seqs=max_seqs,
                              max_batched_tokens=budget, batch=chunk)


def test_greedy_generation_matches_plain(tiny_folders, emu):
    sess = _session(tiny_folders["A"], "A", 64)
    prompts = list(make_requests("A", [7, 16, 33], seed=2).values())
    out = sess.generate(prompts, temp=0, max_tokens=8)
    cfg, W = plain.read_folder(tiny_folders["A"])
    for p, comps in zip(prompts, out):
        assert comps[0].tokens == plain.greedy(cfg, W, p, 8) and comps[0].stop == "length"
    assert sess.engine.cache.pages_in_use() == 0


def test_portions_respect_the_budget_and_decodes_go_first(tiny_folders, emu):
    from hfcpu_b200.engine import Request
    from hfcpu_b200 import SamplingParams
    sess = _session(tiny_folders["B"], "B", 200, budget=48, chunk=32)
    sch = sess.scheduler
    reqs = make_requests("B", [100, 20], seed=1)
    sch.submit(Request("x", reqs["r0"], SamplingParams(temp=0, max_tokens=4)))
    plan = sch.plan()
    assert [len(e.tokens) for e in plan.entries] == [32] and plan.entries[0].want == []
    sch.engine.step(plan.entries)
    plan.requests[0].computed += 32
    sch.submit(Request("y", reqs["r1"], SamplingParams(temp=0, max_tokens=4)))
    plan = sch.plan()                       # x: another portion of 32; y: 16 of its 20 fill the budget of 48
    assert [(e.req, len(e.tokens)) for e in plan.entries] == [("x", 32), ("y", 16)]
    for r in list(sch.running):
        sch.engine.finish_request(r.id)
    sch.running.clear()
    # from scratch: run to the end and look at every step
    sess = _session(tiny_folders["B"], "B", 200, budget=48, chunk=32)
    sch = sess.scheduler
    sch.submit(Request("x", reqs["r0"], SamplingParams(temp=0, max_tokens=6)))
    sch.submit(Request("y", reqs["r1"], SamplingParams(temp=0, max_tokens=6)))
    while sch.has_work():
        plan_tokens = None
        before = {r.id: r.pending for r in sch.running}
        sch.step()
        assert sch.stats["tokens_in"] <= 48 * sch.stats["steps"]
    assert sch.requests["x"].stop == "length" and len(sch.requests["y"].generated) == 6


def test_final_portion_only_asks_for_logits(tiny_folders, emu):
    from hfcpu_b200.engine import Request
    from hfcpu_b200 import SamplingParams
    sess = _session(tiny_folders["A"], "A", 64, budget=16)
    sch = sess.scheduler
    sch.submit(Request("x", list(range(40)), SamplingParams(temp=0, max_tokens=2)))
    wants = []
    while sch.has_work():
        plan = sch.plan()
        wants.append([(len(e.tokens), list(e.want)) for e in plan.entries])
        # undo the plan's side effects by running it through step's path
        logits = sch.engine.step(plan.entries)
        for r, e in zip(plan.requests, plan.entries):
            r.computed += len(e.tokens)
            if e.want:
                r.generated.append(int(torch.argmax(logits[0])))
                if len(r.generated) == 2:
                    sch.running.remove(r)
                    sch.engine.finish_request(r.id)
    assert wants == [[(16, [])], [(16, [])], [(8, [7])], [(1, [0])]]


def test_preemption_keeps_the_sampled_tokens(tiny_folders, emu):
    """With too few pages for all requests to finish together, the newest is put out and recomputed; what
    each request samples (temperature, seeded) is the same as with plenty of pages."""
    prompts = list(make_requests("A", [30, 30, 30], seed=6).values())
    roomy = _session(tiny_folders["A"], "A", 64)
    ref = roomy.generate(prompts, temp=0.9, top_k=0, top_p=1.0, min_p=0.0, seed=5, max_tokens=40)
    tight = _session(tiny_folders["A"], "A", 11)          # 11 pages of 16: three requests of 70 tokens need 15
    got = tight.generate(prompts, temp=0.9, top_k=0, top_p=1.0, min_p=0.0, seed=5, max_tokens=40)
    assert tight.scheduler.stats["preemptions"] > 0
    for a, b in zip(ref, got):
        assert a[0].tokens == b[0].tokens and b[0].stop == "length"
    tight.engine.cache.check()
    assert tight.engine.cache.pages_in_use() == 0


def test_request_that_cannot_fit_fails_alone(tiny_folders, emu):
    sess = _session(tiny_folders["A"], "A", 3)            # 48 tokens of cache in all
    prompts = [list(range(10)), list(range(100)), list(range(12))]
    out = sess.generate(prompts, temp=0, max_tokens=4)
    assert out[0][0].stop == "length" and out[2][0].stop == "length"
    assert out[1][0].stop == "error" and "ENOMEM" in out[1][0].error
    assert sess.engine.cache.pages_in_use() == 0


def test_submit_checks(tiny_folders, emu):
    from hfcpu_b200.engine import Request, RequestError
    from hfcpu_b200 import SamplingParams
    sess = _session(tiny_folders["A"], "A", 64)
    sch = sess.scheduler
    with pytest.raises(RequestError) as e:
        sch.submit(Request("a", [], SamplingParams()))
    assert e.value.code == "EINVAL"
    with pytest.raises(RequestError) as e:
        sch.submit(Request("a", [1] * 256, SamplingParams()))
    assert e.value.code == "ERANGE"
    with pytest.raises(RequestError):
        sch.submit(Request("a", [999], SamplingParams()))
    # max_tokens is clipped to the room the context leaves: stop reason ctx
    out = sess.generate([1] * 250, temp=0, max_tokens=100)
    assert out[0].stop == "ctx" and len(out[0].tokens) == 6


def test_eos_and_fanout_seeds(tiny_folders, emu):
    sess = _session(tiny_folders["A"], "A", 64)
    prompt = list(range(5, 25))
    three = sess.generate(prompt, temp=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=7, max_tokens=12, n=3)
    for i, c in enumerate(three):
        alone = sess.generate(prompt, temp=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=7 + i, max_tokens=12)
        assert alone[0].tokens == c.tokens          # sequence i of a fan-out equals a single run with seed + i
    first = three[0].tokens
    cut = sess.generate(prompt, temp=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=7, max_tokens=12, eos_ids=[first[3]])
    assert cut[0].stop == "eos" and cut[0].tokens == first[:first.index(first[3])]


def test_running_ahead_of_the_host_on_the_stand_in(tiny_folders, emu, monkeypatch):
    """The run loop launches the next steady decode step on token ids the host has not read yet.  Here the sampling
    "kernel" is a host function that hands its ids back as a tensor, so that the bookkeeping (limits, an end token
    that arrives while the next step is in flight, pages given back, the token computed too far being dropped) is
    tested without a GPU: tokens and stop reasons must equal those of the step-by-step loop."""
    import numpy as np
    from hfcpu_b200 import sampling
    from hfcpu_b200.sampling import sample_host

    class HostPending:
        def __init__(self, logits, reqs, host=None):
            rows = logits.float().cpu().numpy()
            self.device = torch.tensor([sample_host(rows[i], r.params, r.rng) for i, r in enumerate(reqs)], dtype=torch.int32)

        def tokens(self):
            return self.device.tolist()

    monkeypatch.setattr(sampling.device, "sample_rows_async", HostPending)
    prompts = list(make_requests("A", [5, 23, 40, 9], seed=9).values())
    ref_sess = _session(tiny_folders["A"], "A", 96)
    ref = ref_sess.generate(prompts, temp=0, max_tokens=20)
    eos = ref[1][0].tokens[7]
    for opts in (dict(temp=0, max_tokens=20), dict(temp=0.9, top_k=30, seed=4, max_tokens=17, n=2),
                 dict(temp=0, max_tokens=20, eos_ids=[eos])):
        outs = []
        for ahead in (False, True):
            sess = _session(tiny_folders["A"], "A", 96)
            sch = sess.scheduler
            if ahead:
                sch.device_sampling = sch.run_ahead = True
                sch._host_ring = [torch.empty(8, dtype=torch.int32) for _ in range(4)]
            outs.append(sess.generate(prompts, **opts))
            assert (sch.stats["steps_ahead"] > 5) == ahead
            sess.engine.cache.check()
            assert sess.engine.cache.pages_in_use() == 0 and sess.engine.slots.free_count == 4
        flat = [[[(c.tokens, c.stop) for c in comps] for comps in o] for o in outs]
        assert flat[0] == flat[1]
    assert any(c.stop == "eos" for comps in outs[1] for c in comps)
