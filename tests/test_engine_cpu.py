"""Host-side logic of the step function against the plain implementation, on the CPU.

The kernels are replaced by the torch stand-in (tests/emu_backend.py); what is under test is the
batch building, the block tables, page reuse, window release and the parts' composition, under
every way of cutting the requests into steps.
"""
import pytest
import torch

import traces
from conftest import BLOCK, TOL, make_requests, plain_logits

LENGTHS = {"A": [7, 16, 33, 100, 70], "B": [1, 19, 64, 130, 200]}


def _engine(folder, name, max_tokens, dtype=torch.float32, max_requests=4):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folder, dtype, "cpu")
    return hfcpu_b200.Engine(model, block_size=BLOCK[name], max_tokens=max_tokens, max_requests=max_requests)


@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed", "one_by_one"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_cuttings_match_plain(tiny_folders, emu, name, family):
    reqs = make_requests(name, LENGTHS[name], seed=3)
    steps = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions,
             "mixed": traces.mixed, "one_by_one": traces.one_by_one}[family](reqs)
    eng = _engine(tiny_folders[name], name, traces.peak_tokens(steps))
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    ref = {r: plain_logits(tiny_folders[name], ids) for r, ids in reqs.items()}
    assert len(got) == sum(len(v) for v in reqs.values())
    bad = traces.first_bad(got, ref, TOL["float32"])
    assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} (error {bad[2]:.3g})"
    assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == eng.max_requests


def test_mixed_reuses_pages(tiny_folders, emu):
    reqs = make_requests("B", [130, 40, 200, 64, 90, 150], seed=9)
    steps = traces.mixed(reqs, max_live=3)
    eng = _engine(tiny_folders["B"], "B", traces.peak_tokens(steps))
    seen = [set() for _ in eng.cache.groups]
    handed_out_again = [False] * len(seen)

    def check():
        eng.cache.check()
        for g in eng.cache.groups:
            now = {p for t in g.tables.values() for p in t if p >= 0}
            handed_out_again[g.index] |= bool((now & seen[g.index]) - getattr(check, f"prev{g.index}", set()))
            setattr(check, f"prev{g.index}", now)
            seen[g.index] |= now
    got = traces.run_in_process(eng, steps, check=check)
    ref = {r: plain_logits(tiny_folders["B"], ids) for r, ids in reqs.items()}
    assert traces.first_bad(got, ref, TOL["float32"]) is None
    assert all(handed_out_again), "the trace was meant to make every group hand pages out again"


def test_step_rejects_bad_entries(tiny_folders, emu):
    from hfcpu_b200 import StepEntry
    from hfcpu_b200.cache import OutOfPages
    eng = _engine(tiny_folders["A"], "A", 64)
    eng.add_request("a")
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", [512], [0])])                  # id outside the vocabulary
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", [1, 2], [2])])                 # wanted place outside the tokens
    with pytest.raises(KeyError):
        eng.step([StepEntry("zz", [1], [0])])
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", [1] * 65, [])])                # more than the pool holds
    assert eng.length("a") == 0 and eng.cache.pages_in_use() == 0
    eng.step([StepEntry("a", [1] * 64, [])])
    assert eng.length("a") == 64


def test_scratch_buffers_keep_and_drop_their_views():
    """A named scratch buffer hands out the same view for the same shape, a buffer that grew hands out views of the
    new storage only, and different shapes of one name share the storage."""
    import torch
    from hfcpu_b200.engine.step import Workspace
    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (4, 8), torch.float32)
    assert ws.get("x", (4, 8), torch.float32) is a and a.shape == (4, 8)
    b = ws.get("x", (2, 8), torch.float32)
    assert b.data_ptr() == a.data_ptr() and b.shape == (2, 8)
    big = ws.get("x", (16, 8), torch.float32)
    assert big.data_ptr() != a.data_ptr()
    again = ws.get("x", (4, 8), torch.float32)
    assert again.data_ptr() == big.data_ptr() and again is not a
    other = ws.get("x", (4, 8), torch.bfloat16)
    assert other.dtype == torch.bfloat16 and other.data_ptr() != again.data_ptr()
    assert a.shape == (4, 8)                                # the outgrown buffer stays alive for graphs that point at it
