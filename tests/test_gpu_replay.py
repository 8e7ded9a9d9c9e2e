"""The engine on the GPU against the plain implementation, under every way of cutting the work.

float32 runs use the float32-stored folders (sharp attention) at 1e-4; bfloat16 runs use the
bfloat16-stored folders at the bfloat16 tolerance, and must also agree with their own whole-prompt
run much more closely than that, since cutting and batching may change results only by rounding.
"""
import os

import pytest
import torch

import traces
from conftest import BLOCK, TINY, TOL, make_requests, plain_logits

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [7, 16, 33, 100, 70], "B": [1, 19, 64, 130, 200], "C": [3, 150, 64, 129, 260]}
FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions,
            "mixed": traces.mixed}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# rows of two cuttings of the same run dtype differ by rounding only
SELF_TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


def folder_for(tiny_folders, name, dtype):
    return tiny_folders[name if dtype == "float32" else name + "16"]


def engine_for(folder, name, dtype, max_tokens, max_requests=4):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folder, DTYPES[dtype], "cuda:0")
    return hfcpu_b200.Engine(model, block_size=BLOCK[name], max_tokens=max_tokens, max_requests=max_requests)


def check_clean(eng):
    from hfcpu_b200 import kernels
    kernels.check_device_errors()
    eng.cache.check()
    assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == eng.max_requests


_WHOLE = {}


def whole_rows(tiny_folders, name, dtype, reqs):
    key = (name, dtype)
    if key not in _WHOLE:
        folder = folder_for(tiny_folders, name, dtype)
        steps = traces.whole(reqs)
        eng = engine_for(folder, name, dtype, traces.peak_tokens(steps))
        _WHOLE[key] = traces.run_in_process(eng, steps)
        check_clean(eng)
    return _WHOLE[key]


@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_cuttings_match_plain(tiny_folders, name, dtype, family):
    folder = folder_for(tiny_folders, name, dtype)
    reqs = make_requests(name, LENGTHS[name], seed=3)
    steps = FAMILIES[family](reqs)
    eng = engine_for(folder, name, dtype, traces.peak_tokens(steps))
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    check_clean(eng)
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    assert len(got) == sum(len(v) for v in reqs.values())
    bad = traces.first_bad(got, ref, TOL[dtype])
    assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} (error {bad[2]:.3g})"
    if family != "whole":
        base = whole_rows(tiny_folders, name, dtype, reqs)
        bad = traces.first_bad(got, {r: torch.stack([base[(r, p)] for p in range(len(ids))]) for r, ids in reqs.items()},
                               SELF_TOL[dtype])
        assert bad is None, f"differs from the whole-prompt run at request {bad[0]} position {bad[1]} ({bad[2]:.3g})"


@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
def test_cuttings_match_plain_with_two_query_tiles_per_cta(tiny_folders, family):
    """The head_dim-128 configuration in bfloat16 with the attention kernel that takes two query tiles per CTA, which
    small prompts do not reach by themselves (it waits for enough CTAs to fill the SMs twice)."""
    from hfcpu_b200 import kernels
    b = kernels.backend()
    old, b.tc2_min_rounds = b.tc2_min_rounds, 0
    try:
        folder = folder_for(tiny_folders, "C", "bfloat16")
        reqs = make_requests("C", [3, 150, 64, 129, 260, 400], seed=5)
        steps = FAMILIES[family](reqs)
        eng = engine_for(folder, "C", "bfloat16", traces.peak_tokens(steps))
        got = traces.run_in_process(eng, steps, check=eng.cache.check)
        check_clean(eng)
        ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
        bad = traces.first_bad(got, ref, TOL["bfloat16"])
        assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} (error {bad[2]:.3g})"
    finally:
        b.tc2_min_rounds = old


@pytest.mark.parametrize("name", ["B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_window(tiny_folders, dtype, name):
    """Token by token from the first token, far past the window (64 in B, 96 in C) and across many pages."""
    folder = folder_for(tiny_folders, name, dtype)
    reqs = make_requests(name, [300], seed=21)
    steps = traces.one_by_one(reqs)
    eng = engine_for(folder, name, dtype, traces.peak_tokens(steps))
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    check_clean(eng)
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    bad = traces.first_bad(got, ref, TOL[dtype])
    assert bad is None, f"first wrong row: position {bad[1]} (error {bad[2]:.3g})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(tiny_folders, name, dtype):
    """Sequences of one, two and three tokens, and the first tokens fed one at a time."""
    folder = folder_for(tiny_folders, name, dtype)
    reqs = make_requests(name, [1, 2, 3, 5], seed=8)
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    for steps in (traces.whole(reqs), traces.one_by_one(reqs), traces.mixed(reqs, prefill_sizes=(2, 1, 3))):
        eng = engine_for(folder, name, dtype, max(64, traces.peak_tokens(steps)))
        got = traces.run_in_process(eng, steps)
        check_clean(eng)
        assert traces.first_bad(got, ref, TOL[dtype]) is None


def test_mixed_hands_pages_out_again(tiny_folders):
    reqs = make_requests("B", [130, 40, 200, 64, 90, 150], seed=9)
    steps = traces.mixed(reqs, max_live=3)
    folder = tiny_folders["B"]
    eng = engine_for(folder, "B", "float32", traces.peak_tokens(steps))
    seen, again, prev = [set() for _ in eng.cache.groups], [False] * len(eng.cache.groups), {}

    def check():
        eng.cache.check()
        for g in eng.cache.groups:
            now = {p for t in g.tables.values() for p in t if p >= 0}
            again[g.index] |= bool((now & seen[g.index]) - prev.get(g.index, set()))
            prev[g.index] = now
            seen[g.index] |= now
    got = traces.run_in_process(eng, steps, check=check)
    check_clean(eng)
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    assert traces.first_bad(got, ref, TOL["float32"]) is None
    assert all(again), "the trace was meant to make every group hand pages out again"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program(tiny_folders, tmp_path, dtype):
    """The same through bin/trace_run over a pipe: mixed requests with a pool so small that pages are used again."""
    name = "B"
    folder = folder_for(tiny_folders, name, dtype)
    reqs = make_requests(name, [130, 40, 200, 64, 90], seed=4)
    steps = traces.mixed(reqs, max_live=4)
    got = traces.run_trace_program(folder, dtype, steps, str(tmp_path / "out"), traces.peak_tokens(steps),
                                   TINY[name]["vocab_size"])
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    assert len(got) == sum(len(v) for v in reqs.values())
    bad = traces.first_bad(got, ref, TOL[dtype])
    assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} (error {bad[2]:.3g})"
