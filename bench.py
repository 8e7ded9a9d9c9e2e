#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on Qwen2.5-7B layer sizes with random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A step is one decode step of a batch of 8 requests that each hold a 2,048-token prompt (maximum
context 4,096).  Prints ONE JSON line: ``value`` = decoded tokens a second over exactly K steps, timed
on the device with CUDA events between synchronisations; ``e2e`` = the same through the Python entry
point (``Session.generate``: host token ids in, host token ids out); ``prefill`` = one 2,048-token prompt;
``roofline`` = bytes a decode step has to read (every weight once, and the cache of the live requests)
over its time against the measured copy bandwidth; ``points`` = decoding at batch 1 and 64.
The engine runs on one GPU only: for N > 1 a line says so and the exit code is 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=3584,
                 num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, vocab_size=152064,
                 max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False,
                 use_sliding_window=False, hidden_act="silu")
PROMPT, CTX_MAX, BLOCK = 2048, 4096, 16
SETTLE_S = 0.5             # pause between the prompts' prefill and the decode steps that are timed
E2E_LEAD = 160             # decode steps of the end-to-end run before its timed ones (about half a second)
REF_DIR = os.path.join(ROOT, "baseline", "_ref", "hf.cpu")     # a copy of the reference's source tree, built by make


def metric_name(batch):
    return f"Qwen2.5-7B bf16: decode tok/s @ batch {batch} ({PROMPT:,}-token prompts, {CTX_MAX:,} max context)"


def run_reference(args):
    """The reference arm: the unmodified reference (a C99 CPU program) built by its own Makefile, run through its own
    command line on the same layer sizes with the same seeded random bf16 weights, written as one of its GGUF files.

        hfcpu --stdin-mode args --model M.gguf ...   with two request lines
        --op generate --prompt-ids "<2,048 ids>" --n 8 --temp 0 --max-tokens W+1     (warm-up)
        --op generate --prompt-ids "<the same>"  --n 8 --temp 0 --max-tokens K+1     (timed by the reference itself)

    ``--n 8`` decodes eight continuations of the prompt together, one forward of eight tokens a step
    (src/ops.c:808-893); the second request starts on the first one's cache of the prompt (src/ops.c:771-776) and its
    ``@genall ms=`` covers exactly K decode steps.  It is a CPU program, so it runs ``--ref-layers`` of the 28 layers
    to stay within minutes; ``config`` names both numbers."""
    import shutil
    import tempfile

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    if args.gpus != 1:
        return unavailable("the reference is a single-process CPU program; it has no multi-GPU form")
    if not os.path.isdir(REF_DIR):
        if not os.path.isdir("/root/reference"):
            return unavailable(f"no copy of the reference's source tree at {os.path.relpath(REF_DIR, ROOT)}")
        shutil.copytree("/root/reference", REF_DIR)
    exe = os.path.join(REF_DIR, "hfcpu")
    if not os.path.exists(exe):
        try:
            r = subprocess.run(["make", "-C", REF_DIR, "hfcpu"], capture_output=True, text=True, timeout=600)
        except (OSError, subprocess.TimeoutExpired) as e:
            return unavailable(f"make -C {os.path.relpath(REF_DIR, ROOT)} hfcpu: {e}")
        if r.returncode != 0 or not os.path.exists(exe):
            return unavailable(f"make -C {os.path.relpath(REF_DIR, ROOT)} hfcpu failed: " + (r.stderr or r.stdout).strip()[-300:].replace("\n", " | "))
    import torch
    import hfcpu_b200
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import RandomSource
    from hfcpu_b200.weights.gguf import write_gguf
    cfg_d = dict(QWEN25_7B, num_hidden_layers=min(args.ref_layers, QWEN25_7B["num_hidden_layers"]))
    cfg = config_from_dict(cfg_d)
    warmup, steps = max(args.warmup, 3), args.steps
    work = tempfile.mkdtemp(prefix="hfb_ref_")
    try:
        gguf = os.path.join(work, "model.gguf")
        write_gguf(gguf, cfg, RandomSource(build_model_specs(cfg), 0, torch.bfloat16, torch.device("cpu")))
        ids = " ".join(map(str, synthetic_prompts(1, PROMPT, cfg.vocab_size, seed=1)[0]))
        script = "".join(f"--op generate --prompt-ids '{ids}' --n {args.batch} --temp 0 --max-tokens {n + 1} --id {tag}\n"
                         for tag, n in (("warm", warmup), ("timed", steps)))
        t0 = time.perf_counter()
        try:
            r = subprocess.run([exe, "--stdin-mode", "args", "--model", gguf, "--ctx-max", str(CTX_MAX), "--batch", "64",
                                "--log-level", "error"], input=script, capture_output=True, text=True, timeout=args.ref_timeout)
        except subprocess.TimeoutExpired:
            return unavailable(f"the reference did not finish {PROMPT} prompt tokens and {warmup + steps} decode steps at "
                               f"{cfg.num_hidden_layers} layers on this machine's CPU within {args.ref_timeout} s")
        wall = time.perf_counter() - t0
        genall = [l for l in r.stdout.splitlines() if l.startswith("@genall")]
        if r.returncode != 0 or len(genall) != 2:
            return unavailable("hfcpu --op generate failed: " + (r.stdout + r.stderr).strip()[-300:].replace("\n", " | "))
        f = dict(kv.split("=", 1) for kv in genall[1].split()[1:])
        ms = float(f["ms"]) / steps
        value = args.batch * steps / (float(f["ms"]) * 1e-3)
        prefill = [l for l in r.stdout.splitlines() if l.startswith("@prefill")][0]
        pf = dict(kv.split("=", 1) for kv in prefill.split()[1:])
    finally:
        shutil.rmtree(work, ignore_errors=True)
    print(json.dumps({
        "metric": metric_name(args.batch), "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random-init weights)", "impl": "reference",
        "device": "cpu", "gpu_launches": 0,
        "config": {"model": "Qwen2.5-7B layer sizes", "layers": cfg.num_hidden_layers, "layers_full": QWEN25_7B["num_hidden_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": PROMPT, "ctx_max": CTX_MAX, "kv_block": 64, "kv_dtype": "f16",
                   "parallelism": "CPU threads (the reference has no GPU path)",
                   "how": "hfcpu --op generate --n 8 --temp 0, timed by its own @genall"},
        "prefill": {"value": float(pf["tok_per_s"]), "tokens": int(pf["tokens"]), "ms": float(pf["ms"])},
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": round(wall, 1)}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# The other two sized workloads the benchmark description names, through the Python entry point (scheduler, chunked
# prompts beside decodes, sampling): `--workload c3` and `--workload c4`.
WORKLOADS = {
    "c3": dict(name="Qwen2.5-0.5B layer sizes: 32 requests, prompts uniform in [1, 1024], 128 new tokens each, 256-token "
                    "prompt portions beside decodes, temperature 0.7",
               cfg=dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2,
                        intermediate_size=4864, vocab_size=151936, tie_word_embeddings=True, rms_norm_eps=1e-6),
               requests=32, prompt=(1, 1024), new=128, chunk=256, ctx_max=2048, temp=0.7),
    "c4": dict(name="Qwen2.5-32B layer sizes: 16 requests, 4,096-token prompts, 128 new tokens each, greedy, 8,192 max context",
               cfg=dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                        intermediate_size=27648, vocab_size=152064, tie_word_embeddings=False, rms_norm_eps=1e-5),
               requests=16, prompt=(4096, 4096), new=128, chunk=2048, ctx_max=8192, temp=0.0),
}


def run_workload(args):
    """One of WORKLOADS end to end through Session.generate, host ids in and out: one JSON line with the wall-clock
    time, the tokens a second over the whole run, and over the stretch after every request has its first token."""
    import torch
    import hfcpu_b200
    from hfcpu_b200.config import config_from_dict
    w = WORKLOADS[args.workload]
    cfg_d = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", max_position_embeddings=32768, rope_theta=1e6,
                 use_sliding_window=False, hidden_act="silu", **w["cfg"])
    layers_full = cfg_d["num_hidden_layers"]
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfg_d)
    torch.cuda.set_device(0)
    model = hfcpu_b200.random_model(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    g = torch.Generator().manual_seed(11)
    lens = torch.randint(w["prompt"][0], w["prompt"][1] + 1, (w["requests"],), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    sess = hfcpu_b200.Session(model, kv_block=BLOCK, max_seqs=w["requests"], ctx_max=w["ctx_max"],
                              kv_pages=w["requests"] * (w["ctx_max"] // BLOCK + 1), max_batched_tokens=max(w["chunk"], w["requests"]),
                              batch=w["chunk"])
    runs = []
    for rep in range(2):                                     # the first run warms up (graphs, buffers); the second is the record
        first, stamps = {}, []

        def on_event(ev):
            if hasattr(ev, "token"):
                now = time.perf_counter()
                first.setdefault(ev.req, now)
                stamps.append(now)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = sess.generate(prompts, temp=w["temp"], seed=5, max_tokens=w["new"], eos_ids=[], on_event=on_event, prefix_cache=False)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        new = sum(len(c[0].tokens) for c in out)
        t_all_first = max(first.values())
        after = sum(1 for t in stamps if t > t_all_first)
        runs.append(dict(seconds=round(t1 - t0, 4), new_tokens=new, prompt_tokens=sum(lens),
                         tokens_per_s=round((sum(lens) + new) / (t1 - t0), 1), new_tokens_per_s=round(new / (t1 - t0), 1),
                         seconds_to_all_first_tokens=round(t_all_first - t0, 4),
                         decode_tokens_per_s=round(after / max(t1 - t_all_first, 1e-9), 1)))
    from hfcpu_b200 import kernels
    kernels.check_device_errors()
    print(json.dumps({"workload": args.workload, "name": w["name"], "impl": "engine", "dtype": "bf16",
                      "data": "synthetic (seeded uniform token ids, random-init weights)",
                      "config": {"layers": cfg.num_hidden_layers, "layers_full": layers_full, "requests": w["requests"],
                                 "chunk": w["chunk"], "ctx_max": w["ctx_max"], "temp": w["temp"], "kv_block": BLOCK},
                      **runs[-1], "first_run_seconds": runs[0]["seconds"]}))
    return 0


def synthetic_prompts(batch, n, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, n), generator=g).tolist()


def prefill_requests(engine, prompts, tag):
    """Prefill every prompt (one request a step) and return each request's first greedy token."""
    import torch
    from hfcpu_b200 import StepEntry
    first = []
    for b, ids in enumerate(prompts):
        engine.add_request((tag, b))
        logits = engine.step([StepEntry((tag, b), ids, [len(ids) - 1])])
        first.append(int(torch.argmax(logits[0])))
    return first


def time_decode(engine, batch, steps, warmup, vocab, seed, sampler=None):
    """(ms per step, bytes of cache read per step at the middle of the run, launches per step)."""
    import torch
    from hfcpu_b200 import StepEntry, kernels
    tag = f"dec{batch}"
    toks = prefill_requests(engine, synthetic_prompts(batch, PROMPT, vocab, seed), tag)
    outs = [torch.empty(batch, dtype=torch.int32, device=engine.device) for _ in range(2)]
    entries = [StepEntry((tag, b), [0], [0]) for b in range(batch)]
    prev = torch.tensor(toks, dtype=torch.int32, device=engine.device)
    n_done = 0

    def one_step():
        # the ids the arg-max kernel wrote feed the next step on the device: the GPU never waits for the host
        nonlocal prev, n_done
        logits = engine.step(entries, token_source=prev)
        prev = outs[n_done & 1]
        kernels.argmax(logits, prev)
        n_done += 1

    # The prompts' prefill leaves the GPU at the clocks of its power cap for some hundred milliseconds; the numbers
    # here are those of decoding, so the GPU gets half a second to come back before the warm-up steps.
    torch.cuda.synchronize()
    time.sleep(SETTLE_S)
    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    launches0 = kernels.backend().launches
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = (kernels.backend().launches - launches0) / steps
    ctx_mid = PROMPT + warmup + steps // 2
    for b in range(batch):
        engine.finish_request((tag, b))
    return ms, ctx_mid, launches


def print_timeline(args, engine, vocab):
    """One decode step of the batch (after seven warm ones), or one prompt of PROMPT tokens, kernel by kernel."""
    import torch
    from hfcpu_b200 import StepEntry, kernels
    from hfcpu_b200.kernels import timeline
    if args.timeline == "decode":
        tag = "tl"
        toks = prefill_requests(engine, synthetic_prompts(args.batch, PROMPT, vocab, 1), tag)
        out = torch.empty(args.batch, dtype=torch.int32, device=engine.device)
        for s in range(8):
            if s == 7:
                torch.cuda.synchronize()
                timeline.start()
            logits = engine.step([StepEntry((tag, b), [toks[b]], [0]) for b in range(args.batch)])
            kernels.argmax(logits, out)
            toks = out.tolist()
    else:
        for i, ids in enumerate(synthetic_prompts(3, PROMPT, vocab, 5)):
            engine.add_request(("tl", i))
            if i == 2:
                torch.cuda.synchronize()
                timeline.start()
            engine.step([StepEntry(("tl", i), ids, [PROMPT - 1])])
            torch.cuda.synchronize()
            engine.finish_request(("tl", i))
    records = timeline.take()
    print(timeline.format_marks(records) if args.marks else timeline.format_rows(timeline.kernels(records)))
    return 0


def main():
    global PROMPT, CTX_MAX
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=192)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the 28 of the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt length (the record uses 2,048; others are for profiling)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the end-to-end run")
    ap.add_argument("--timeline", choices=["decode", "prefill"], help="print the kernel timeline of one step instead of the "
                    "record (needs a library built with HFB_NVCC_EXTRA=-DHFB_TRACE; see hfcpu_b200/kernels/timeline.py)")
    ap.add_argument("--marks", action="store_true", help="with --timeline: every logged mark, not one row per kernel")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), help="run one of the other sized workloads end to end through "
                    "Session.generate instead of the record (c3: 0.5B sizes, mixed chunked prompts and decodes; c4: 32B sizes)")
    ap.add_argument("--ref-layers", type=int, default=28, help="layers the reference arm runs (it is a CPU program)")
    ap.add_argument("--ref-timeout", type=int, default=1500, help="seconds the reference arm may take")
    args = ap.parse_args()
    if args.prompt != PROMPT:
        PROMPT = args.prompt
        CTX_MAX = max(CTX_MAX, 2 * PROMPT)

    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload:
        return run_workload(args)
    warmup = max(args.warmup, 3)

    import torch
    import hfcpu_b200
    from hfcpu_b200 import StepEntry, kernels
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.engine import measure

    cfg_d = dict(QWEN25_7B)
    layers_full = cfg_d["num_hidden_layers"]
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfg_d)
    V = cfg.vocab_size
    torch.cuda.set_device(0)
    kernels.backend()
    model = hfcpu_b200.random_model(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    max_b = max(64, args.batch)
    pages = max_b * ((PROMPT + max(warmup, E2E_LEAD) + args.steps + 64 + BLOCK - 1) // BLOCK + 1)
    engine = hfcpu_b200.Engine(model, block_size=BLOCK, num_pages=pages, max_requests=max_b, ctx_max=CTX_MAX)
    pk, pk_src = measure.load_peaks(ROOT)
    if args.timeline:
        return print_timeline(args, engine, V)

    # ---- prefill: one prompt of 2,048 tokens, eight times over ----------------------------------------------
    # The first two warm up.  The next three are each timed alone, after a pause, as the peak they are set against
    # was (a burst: the best of ten products); the last three run back to back.  `ms` and `frac` are the median of
    # the six; the medians of the three alone and of the three in a row are reported beside them (they differ by a
    # per cent or two either way: a pause lets the power budget recover, and lets the clocks fall).
    pre_ms = []
    for i, ids in enumerate(synthetic_prompts(8, PROMPT, V, seed=100)):
        engine.add_request(("pre", i))
        torch.cuda.synchronize()
        if 2 <= i <= 5:
            time.sleep(SETTLE_S)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step([StepEntry(("pre", i), ids, [PROMPT - 1])])
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
        engine.finish_request(("pre", i))
    kernels.check_device_errors()
    pre = statistics.median(pre_ms[2:])
    L, E, F = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
    flops = measure.step_flops(model, [PROMPT], [PROMPT], 1)
    prefill = {"value": round(PROMPT / pre * 1e3, 1), "tokens": PROMPT, "ms": round(pre, 3),
               "frac": round(flops / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "tflop": round(flops / 1e12, 2),
               "peak_tflops": pk["bf16_tflops"], "peak_source": pk_src, "best_ms": round(min(pre_ms[2:]), 3),
               "alone_ms": round(statistics.median(pre_ms[2:5]), 3), "back_to_back_ms": round(statistics.median(pre_ms[5:]), 3),
               "timing": "median of six prompts: three each timed alone after a pause (alone_ms), three in a row (back_to_back_ms)"}

    # ---- decode: the default batch, timed with clocks sampled ------------------------------------------
    sampler = ClockSampler()
    ms, ctx_mid, launches = time_decode(engine, args.batch, args.steps, warmup, V, seed=1, sampler=sampler)
    clocks = sampler.stop()
    kernels.check_device_errors()          # a number from a step whose kernels gave up is no number
    value = args.batch / ms * 1e3
    step_bytes = measure.decode_step_bytes(engine, [ctx_mid] * args.batch)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk_src,
                "bytes_per_step": step_bytes}

    points, e2e = {}, None
    if not args.no_points:
        for b in (1, 64):
            pms, _, _ = time_decode(engine, b, args.steps, warmup, V, seed=2 + b)
            points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
        kernels.check_device_errors()
        # ---- end to end through the Python entry point: host ids in, host ids out -----------------------
        del engine
        torch.cuda.empty_cache()
        # all prompts are prefilled in the first step, so that every later step decodes exactly `batch` tokens
        sess = hfcpu_b200.Session(model, kv_block=BLOCK, kv_pages=pages, max_seqs=max_b, ctx_max=CTX_MAX,
                                  max_batched_tokens=args.batch * PROMPT)
        prompts = synthetic_prompts(args.batch, PROMPT, V, seed=7)
        stamps = []
        # One call prefills and decodes, so the first decode steps run at the clocks the prefill's power cap left:
        # the call decodes E2E_LEAD steps beyond the warm-up first, and its last K steps are the timed ones.
        lead = max(warmup, E2E_LEAD)
        sess.generate(prompts, temp=0, max_tokens=lead + args.steps + 1, eos_ids=[],
                      on_event=lambda ev: stamps.append(time.perf_counter()) if hasattr(ev, "token") else None)
        # token events arrive batch by batch; time the last K decode steps
        t_first = stamps[args.batch * (lead + 1) - 1]
        t_last = stamps[-1]
        e2e_value = args.batch * args.steps / (t_last - t_first)
        meta_ints = 3 * args.batch + (args.batch + 1) + 3 * args.batch + args.batch * (1 + (CTX_MAX // BLOCK // 2))
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * meta_ints + 20 * args.batch,
               "d2h_bytes_per_step": 4 * args.batch}

    line = {
        "metric": metric_name(args.batch),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random-init weights)",
        "impl": "engine",
        "config": {"model": "Qwen2.5-7B layer sizes", "layers": cfg.num_hidden_layers, "layers_full": layers_full,
                   "hidden": E, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": F, "vocab": V, "global_batch": args.batch, "seq_len": PROMPT,
                   "ctx_max": CTX_MAX, "kv_block": BLOCK, "kv_dtype": "bf16", "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights read every step)"},
        "prefill": prefill, "roofline": roofline, "points": points, "clocks": clocks,
        "gpu_launches": int(round(launches * args.steps)), "launches_per_step": round(launches, 1),
    }
    if e2e:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
