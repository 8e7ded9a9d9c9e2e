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


def _drain(sch, check=True):
    while sch.has_work():
        sch.step()
        if check:
            sch.engine.cache.check()


def test_continuations_of_one_prompt_start_on_its_pages(tiny_folders, emu):
    """Requests with the same prompt: the first computes it, the others wait for it and start on its full pages;
    what every one of them samples is what it samples without sharing."""
    from hfcpu_b200.engine import Request
    from hfcpu_b200 import SamplingParams
    prompt = make_requests("A", [45], seed=5)["r0"]
    bs = BLOCK["A"]
    results = {}
    for share in (False, True):
        sess = _session(tiny_folders["A"], "A", 64, budget=16)
        sch = sess.scheduler
        sch.share_prefixes = share
        for i in range(3):
            sch.submit(Request(("n", i), prompt, SamplingParams(temp=0.9, top_k=8, seed=11 + i, max_tokens=6)))
        _drain(sch)
        results[share] = ([sch.requests[("n", i)].generated for i in range(3)], dict(sch.stats))
        assert sess.engine.cache.pages_in_use() == 0
    assert results[True][0] == results[False][0]
    shared = (len(prompt) - 1) // bs * bs
    assert results[True][1]["tokens_shared"] == 2 * shared and results[False][1]["tokens_shared"] == 0
    assert results[False][1]["tokens_in"] - results[True][1]["tokens_in"] == 2 * shared


def test_a_request_starts_on_a_running_request_with_the_same_first_tokens(tiny_folders, emu):
    from hfcpu_b200.engine import Request
    from hfcpu_b200 import SamplingParams
    a = make_requests("B", [60], seed=7)["r0"]
    b = a[:37] + make_requests("B", [20], seed=8)["r0"]            # the same first 37 tokens, then its own
    bs = BLOCK["B"]
    outs = {}
    for share in (False, True):
        sess = _session(tiny_folders["B"], "B", 200, budget=32)
        sch = sess.scheduler
        sch.share_prefixes = share
        sch.submit(Request("a", a, SamplingParams(temp=0, max_tokens=12)))
        sch.step(); sch.step(); sch.step()                         # a is decoding when b arrives
        sch.submit(Request("b", b, SamplingParams(temp=0, max_tokens=5)))
        _drain(sch)
        outs[share] = (sch.requests["a"].generated, sch.requests["b"].generated, sch.requests["b"].shared)
        assert sess.engine.cache.pages_in_use() == 0
    assert outs[True][:2] == outs[False][:2]
    assert outs[True][2] == 37 // bs * bs and outs[False][2] == 0


def test_pages_kept_of_the_previous_request(tiny_folders, emu):
    """keep_cache: the pages of a finished request stay until the next request has started, on them if its first
    tokens are the same; they go at once when pages are short."""
    from hfcpu_b200.engine import Request
    from hfcpu_b200 import SamplingParams
    bs = BLOCK["A"]
    first = make_requests("A", [30], seed=3)["r0"]
    sess = _session(tiny_folders["A"], "A", 64, budget=64)
    sch = sess.scheduler
    sch.submit(Request(1, first, SamplingParams(temp=0, max_tokens=10), keep_cache=True))
    _drain(sch)
    said = sch.requests[1].generated
    assert sch.retained is sch.requests[1] and sess.engine.cache.pages_in_use() > 0
    # the next turn: the whole exchange so far, and more
    follow = first + said + make_requests("A", [9], seed=4)["r0"]
    sch.submit(Request(2, follow, SamplingParams(temp=0, max_tokens=6)))
    _drain(sch)
    cached = (len(first) + len(said) - 1)                          # the last sampled token was never run
    assert sch.requests[2].shared == min(cached, len(follow) - 1) // bs * bs > 0
    assert sch.retained is None and sess.engine.cache.pages_in_use() == 0
    fresh = _session(tiny_folders["A"], "A", 64, budget=64)
    assert fresh.generate([follow], temp=0, max_tokens=6)[0][0].tokens == sch.requests[2].generated
    # kept pages give way: a pool that cannot hold both
    sess = _session(tiny_folders["A"], "A", (40 + bs - 1) // bs + 1, budget=64)
    sch = sess.scheduler
    sch.submit(Request(1, first, SamplingParams(temp=0, max_tokens=8), keep_cache=True))
    _drain(sch)
    assert sch.retained is not None
    other = make_requests("A", [36], seed=9)["r0"]
    sch.submit(Request(2, other, SamplingParams(temp=0, max_tokens=3)))
    _drain(sch)
    assert sch.requests[2].stop == "length" and sch.requests[2].shared == 0 and sch.retained is None
    assert sess.engine.cache.pages_in_use() == 0


def test_a_request_waits_only_for_the_tokens_it_shares(tiny_folders, emu):
    """Both arrive together; the second shares 37 tokens with the first, which needs several steps for its prompt:
    the second waits until those tokens (whole blocks of them) are computed, not for the whole prompt."""
    from hfcpu_b200.engine import Request
    from hfcpu_b200 import SamplingParams
    from hfcpu_b200.engine.scheduler import Scheduler
    assert Scheduler._common([1, 2, 3, 4], [1, 2, 9, 4], 4) == 2 and Scheduler._common([1, 2], [1, 2, 3], 5) == 2
    assert Scheduler._common(list(range(2000)), list(range(1500)) + [0] * 500, 2000) == 1500
    a = make_requests("B", [60], seed=7)["r0"]
    b = a[:37] + make_requests("B", [20], seed=8)["r0"]
    bs = BLOCK["B"]
    sess = _session(tiny_folders["B"], "B", 200, budget=24, chunk=16)   # a takes 16 tokens a step, 8 are left for b
    sch = sess.scheduler
    sch.submit(Request("a", a, SamplingParams(temp=0, max_tokens=4)))
    sch.submit(Request("b", b, SamplingParams(temp=0, max_tokens=4)))
    admitted_at = None
    for step in range(1, 40):
        sch.step()
        sch.engine.cache.check()
        if admitted_at is None and sch.requests["b"].status != "waiting":
            admitted_at = step
            assert sch.requests["a"].computed < len(a)            # a's own prompt is not through yet
        if not sch.has_work():
            break
    share = 37 // bs * bs
    assert sch.requests["b"].shared == share
    assert admitted_at == share // 16 + 1                          # the step after a has computed the shared blocks
    assert sess.engine.cache.pages_in_use() == 0
    alone = _session(tiny_folders["B"], "B", 200, budget=16)
    assert alone.generate([b], temp=0, max_tokens=4)[0][0].tokens == sch.requests["b"].generated


def test_timeouts_end_requests_and_give_their_pages_back(tiny_folders, emu, monkeypatch):
    """--timeout: past the limit a request that has its first token ends with stop=timeout (src/ops.c:829-833); one
    that is still computing its prompt fails with ECANCEL (src/ops.c:790-791).  The clock is the test's."""
    import hfcpu_b200.engine.scheduler as S
    from hfcpu_b200 import SamplingParams
    from hfcpu_b200.engine import FinishEvent, Request
    now = [100.0]
    monkeypatch.setattr(S.time, "perf_counter", lambda: now[0])
    sess = _session(tiny_folders["A"], "A", 64, budget=16, chunk=8)
    sch = sess.scheduler
    reqs = make_requests("A", [6, 40, 5], seed=9)
    sch.submit(Request("fast", reqs["r0"], SamplingParams(temp=0, max_tokens=50), timeout=5.0))
    sch.submit(Request("slow", reqs["r1"], SamplingParams(temp=0, max_tokens=50), timeout=5.0))
    sch.submit(Request("free", reqs["r2"], SamplingParams(temp=0, max_tokens=3)))                 # no limit of its own
    events = []
    for _ in range(2):                      # "fast" has its first token, "slow" is two portions into its prompt
        now[0] += 1.0
        events += sch.step()
    fast, slow = sch.requests["fast"], sch.requests["slow"]
    assert fast.generated and slow.computed < len(slow.prompt) and not slow.generated
    now[0] += 10.0
    events += sch.step()
    ends = {e.req: e for e in events if isinstance(e, FinishEvent)}
    assert ends["fast"].stop == "timeout" and ends["fast"].error is None and len(fast.generated) >= 1
    assert ends["slow"].stop == "error" and ends["slow"].error.startswith("ECANCEL")
    events += sch.run()
    assert sch.requests["free"].stop == "length" and len(sch.requests["free"].generated) == 3
    assert sess.engine.cache.pages_in_use() == 0 and not sess.engine.live_requests()
    sess.engine.cache.check()


def test_cancel_between_steps(tiny_folders, emu):
    """Scheduler.cancel: a running request and a waiting one both end with stop=cancel at the next step; the others
    go on and generate what they would have generated alone."""
    from hfcpu_b200 import SamplingParams
    from hfcpu_b200.engine import FinishEvent, Request
    sess = _session(tiny_folders["A"], "A", 64, max_seqs=2)
    sch = sess.scheduler
    reqs = make_requests("A", [9, 12, 7], seed=5)
    for name, ids in zip("abc", reqs.values()):
        sch.submit(Request(name, ids, SamplingParams(temp=0, max_tokens=6)))
    sch.step()
    assert [r.id for r in sch.running] == ["a", "b"] and [r.id for r in sch.waiting] == ["c"]
    sch.cancel("a")
    sch.cancel("c")
    events = sch.run()
    ends = {e.req: e.stop for e in events if isinstance(e, FinishEvent)}
    assert ends == {"a": "cancel", "c": "cancel", "b": "length"}
    cfg, W = plain.read_folder(tiny_folders["A"])
    assert sch.requests["b"].generated == plain.greedy(cfg, W, reqs["r1"], 6)
    assert len(sch.requests["a"].generated) <= 1 and not sch.requests["c"].generated
    assert sess.engine.cache.pages_in_use() == 0 and not sess.engine.live_requests()


def test_a_step_that_raises_leaves_nothing_behind(tiny_folders, emu):
    """When the engine's step fails, the call's requests are ended and their pages returned, so that the next call on
    the same session runs alone and gives what it gives on a fresh one."""
    sess = _session(tiny_folders["A"], "A", 64)
    prompts = list(make_requests("A", [7, 16], seed=2).values())
    real, calls = sess.engine.model.forward, [0]

    def failing(ctx):
        calls[0] += 1
        if calls[0] == 3:
            raise RuntimeError("a kernel met a device-side wait that ran out")
        return real(ctx)
    sess.engine.model.forward = failing
    with pytest.raises(RuntimeError, match="ran out"):
        sess.generate(prompts, temp=0, max_tokens=8)
    sess.engine.model.forward = real
    assert not sess.scheduler.has_work() and not sess.engine.live_requests() and sess.engine.cache.pages_in_use() == 0
    out = sess.generate(prompts[0], temp=0, max_tokens=5)
    cfg, W = plain.read_folder(tiny_folders["A"])
    assert out[0].tokens == plain.greedy(cfg, W, prompts[0], 5)
