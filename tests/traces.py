"""Traces: ways of cutting the same requests into steps, and two ways of running a trace.

A trace is a list of steps; a step is ``{"step": n, "entries": [{"id", "tokens", "want"}], "end": [...]}``,
the format ``bin/trace_run`` reads.  Every builder below asks for the logits at *every* position, so
that any cutting can be compared with the plain implementation position by position.
"""
import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _entry(req, tokens, first_pos):
    return {"id": req, "tokens": list(tokens), "want": list(range(len(tokens))), "_pos": first_pos}


def whole(reqs):
    """Each request alone and whole: one step per request."""
    return [{"step": i, "entries": [_entry(r, ids, 0)], "end": [r]} for i, (r, ids) in enumerate(reqs.items())]


def tail_one_by_one(reqs, tail=32):
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for r, ids in reqs.items():
        head = max(1, len(ids) - tail)
        cuts = [(0, head)] + [(p, p + 1) for p in range(head, len(ids))]
        for k, (a, b) in enumerate(cuts):
            steps.append({"step": len(steps), "entries": [_entry(r, ids[a:b], a)], "end": [r] if b == len(ids) else []})
    return steps


def one_by_one(reqs):
    """Long decoding: every token of a request in a step of its own."""
    return tail_one_by_one(reqs, tail=10 ** 9)


def portions(reqs, sizes=(32, 7, 16, 2, 5, 64, 3, 2, 11)):
    """Portions of changing size, down to two tokens."""
    steps, k = [], 0
    for r, ids in reqs.items():
        a = 0
        while a < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - a)
            if len(ids) - a - n == 1:      # never leave a single token for a portion of its own
                n += 1
            k += 1
            steps.append({"step": len(steps), "entries": [_entry(r, ids[a:a + n], a)],
                          "end": [r] if a + n == len(ids) else []})
            a += n
    return steps


def mixed(reqs, max_live=4, seed=0, prefill_sizes=(24, 2, 9, 40, 5, 17), decode_after=0.6):
    """Up to ``max_live`` requests at a time; each feeds the first part of its tokens in portions and the
    rest one token a step, so portions of some run beside single tokens of others; a request may sit
    a step out; finished requests make room for waiting ones (their pages are handed out again)."""
    rnd = random.Random(seed)
    waiting = list(reqs)
    live, fed, steps, k = [], {r: 0 for r in reqs}, [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, end = [], []
        for r in list(live):
            ids = reqs[r]
            if len(live) > 1 and rnd.random() < 0.2:
                continue
            a = fed[r]
            if a >= int(len(ids) * decode_after) and a > 0:
                n = 1
            else:
                n = min(prefill_sizes[k % len(prefill_sizes)], len(ids) - a)
                k += 1
            entries.append(_entry(r, ids[a:a + n], a))
            fed[r] = a + n
            if fed[r] == len(ids):
                end.append(r)
                live.remove(r)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def peak_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each rounded up to a multiple of ``round_to``."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return peak


def run_in_process(engine, steps, check=None):
    """Run a trace on an Engine; returns {(request, position): float32 logits row on the CPU}."""
    from hfcpu_b200 import StepEntry
    out = {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not engine.has_request(e["id"]):
                engine.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = engine.step(entries)
        if logits is not None:
            rows = logits.detach().float().cpu()
            o = 0
            for e in s["entries"]:
                for w in e["want"]:
                    out[(e["id"], e["_pos"] + w)] = rows[o].clone()
                    o += 1
        for r in s["end"]:
            engine.finish_request(r)
        if check:
            check()
    return out


def run_trace_program(model_dir, dtype, steps, out_dir, max_tokens, vocab, block_size=None, env=None):
    """Run a trace through ``bin/trace_run`` over a pipe, step by step, waiting for each ``done`` line."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    if block_size:
        cmd += ["--block-size", str(block_size)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    out = {}
    try:
        for s in steps:
            rec = {"step": s["step"], "entries": [{k: v for k, v in e.items() if not k.startswith("_")}
                                                   for e in s["entries"]], "end": s["end"]}
            p.stdin.write(json.dumps(rec) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run answered {line!r}"
            if any(e["want"] for e in s["entries"]):
                rows = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(-1, vocab)
                o = 0
                for e in s["entries"]:
                    for w in e["want"]:
                        out[(e["id"], e["_pos"] + w)] = torch.from_numpy(rows[o].copy())
                        o += 1
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    return out


def worst_error(got, ref):
    """max over rows of max|a-b| / max|b|, and the (request, position) where it occurs."""
    worst, where = 0.0, None
    for (r, pos), row in got.items():
        b = ref[r][pos]
        e = float((row.double() - b.double()).abs().max() / b.double().abs().max())
        if e > worst or where is None:
            worst, where = max(worst, e), (r, pos) if e >= worst else where
    return worst, where


def first_bad(got, ref, tol):
    """The first (request, position) whose row is off by more than ``tol``: where to start looking."""
    for (r, pos) in sorted(got, key=lambda k: (str(k[0]), k[1])):
        b = ref[r][pos]
        e = float((got[(r, pos)].double() - b.double()).abs().max() / b.double().abs().max())
        if e > tol:
            return r, pos, e
    return None
