"""The command line: one resident process, requests on stdin, events on stdout, logs on stderr.

Modes of stdin, controls, events and exit codes follow the reference (src/main.c:54-199,
docs/PROTOCOL.md): ``prompts`` = records separated by a byte, each with an optional option line ended by
0x1f; ``args`` = one request per line written as options, with ``!quit``, ``!stats``, ``!cancel``; ``none``
= one request from the command line.  Every request answers ``@begin id= op=`` ... ``@done status=ok|error
[code= msg=] ms=`` (src/ops.c:1042-1073).  Exit codes: 0, 1 (failed request in mode none, or stdout
closed), 2 (startup option error), 130 (interrupted).
"""
from __future__ import annotations

import os
import signal
import sys
import time
from typing import Any, Dict, List, Optional

from . import opts as O
from .proto import EventWriter, RecordReader

LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3}


class Failure(Exception):
    def __init__(self, code: str, msg: str):
        super().__init__(msg)
        self.code, self.msg = code, msg


class App:
    device = "cuda:0"               # where --random-weights models are made (the engine has no CPU path)

    def __init__(self, session_opts: Dict[str, Any], out: EventWriter):
        self.o, self.out = session_opts, out
        self.n_requests = self.n_errors = 0
        self.session = None             # resident model + engine, reloaded when the model path or its file changes
        self.session_key = None
        self.interrupted = False
        self.cancel_requested = False
        self._serial = 0

    def log(self, level: str, **kv) -> None:
        if LEVELS[level] <= LEVELS[self.o["log_level"]]:
            from .proto import quote
            print(level + " " + " ".join(f"{k}={quote(str(v))}" for k, v in kv.items()), file=sys.stderr, flush=True)

    # ---- requests -----------------------------------------------------------------------------
    def run_request(self, eff: Dict[str, Any], body: Optional[bytes]) -> bool:
        self.n_requests += 1
        self._serial += 1
        rid = eff["id"] if eff["id"] is not None else str(self._serial)
        op = eff["op"] or "generate"
        self.out.event("begin", id=rid, op=op)
        t0 = time.perf_counter()
        try:
            handler = {"echo": self.op_echo, "generate": self.op_generate, "bench": self.op_bench,
                       "inspect": self.op_inspect}.get(op)
            if handler is None:
                raise Failure("ENOTSUP" if op in ("doctor", "tokenize") else "EINVAL",
                              f"operation '{op}' is not supported (generate | bench | inspect | echo)")
            handler(eff, body)
        except Failure as f:
            self.n_errors += 1
            self.out.event("done", status="error", code=f.code, msg=f.msg, ms=f"{(time.perf_counter() - t0) * 1e3:.1f}")
            return False
        self.out.event("done", status="ok", ms=f"{(time.perf_counter() - t0) * 1e3:.1f}")
        return True

    def failed_request(self, code: str, msg: str) -> None:
        self.n_requests += 1
        self.n_errors += 1
        self._serial += 1
        self.out.event("begin", id=str(self._serial), op="none")
        self.out.event("done", status="error", code=code, msg=msg, ms="0.0")

    def op_echo(self, eff, body):
        # every option as "@opt key= value=" (src/ops.c:146-159, src/opts.c:446-463), then the texts as payloads
        for o in O.OPTIONS:
            v = eff[o.key]
            if v is None:
                v = ""
            elif isinstance(v, bool):
                v = int(v)
            elif isinstance(v, float):
                v = f"{v:g}"
            self.out.event("opt", key=o.name, value=v)
        self.out.payload("system", (eff["system"] or "").encode())
        self.out.payload("prompt", body if body is not None else (eff["prompt"] or "").encode())

    def _reject_text(self, eff, body):
        for o in O.OPTIONS:
            if o.note == "text" and o.kind != O.BOOL and eff[o.key] is not None:
                raise Failure("ENOTSUP", f"--{o.name} needs a tokenizer, which this engine does not have; use --prompt-ids")
        if body:
            raise Failure("ENOTSUP", "a text prompt needs a tokenizer, which this engine does not have; use --prompt-ids")

    def _random_model(self):
        """The model of --random-weights CONFIG.json: the configuration's class from the registry, weights drawn on
        the device from --weights-seed (the role of the reference's tools/mkmodel.pl:104-119, without a file)."""
        import json
        import torch
        import hfcpu_b200
        from hfcpu_b200.config import config_from_dict
        path = self.o["random_weights"]
        try:
            with open(path) as f:
                d = json.load(f)
        except OSError as e:
            raise Failure("EIO", f"{path}: {e.strerror}") from None
        except ValueError as e:
            raise Failure("EFORMAT", f"{path}: not valid JSON ({e})") from None
        if not isinstance(d, dict):
            raise Failure("EFORMAT", f"{path}: top level must be an object")
        seed = self.o["weights_seed"] if self.o["weights_seed"] is not None else self.o["seed"]
        dtype = torch.float32 if self.o["dtype"] in ("fp32", "float32") else torch.bfloat16
        return hfcpu_b200.random_model(config_from_dict(d), seed=int(seed), dtype=dtype, device=self.device,
                                       std=float(self.o["weights_std"]))

    def _resident(self, eff):
        path = eff["model"]
        random = self.o["random_weights"]
        if not path and not random:
            raise Failure("EINVAL", f"{eff['op'] or 'generate'} needs --model PATH (or --random-weights CONFIG.json)")
        import hfcpu_b200
        from hfcpu_b200.config import ConfigError, UnsupportedError
        from hfcpu_b200.weights import WeightError, WeightFormatError
        if not path:
            path = "random:" + os.path.abspath(random)
        from hfcpu_b200.weights import find_weight_files
        try:
            files = ([random] if path.startswith("random:") else
                     find_weight_files(path)[0] if os.path.isdir(path) else [path])
            key = (path,) + tuple((f, os.stat(f).st_size, os.stat(f).st_mtime_ns) for f in files)
        except (OSError, WeightFormatError):
            key = (path, -1, -1)
        if self.session is not None and self.session_key == key:
            return self.session
        self.session = None
        eos = None
        if self.o["eos_ids"]:
            eos = parse_ids(self.o["eos_ids"], 1 << 31)
        try:
            self.session = hfcpu_b200.Session(
                self._random_model() if path.startswith("random:") else path, dtype=self.o["dtype"], ctx_max=int(self.o["ctx_max"]), batch=int(self.o["batch"]),
                kv_block=self.o["kv_block"], kv_pages=int(self.o["kv_pages"]), kv_mem=int(self.o["kv_mem"]),
                max_seqs=self.o["max_seqs"], max_batched_tokens=self.o["max_batched_tokens"], eos_ids=eos)
        except UnsupportedError as e:
            raise Failure("ENOTSUP", str(e)) from None
        except (ConfigError, WeightError, WeightFormatError) as e:
            raise Failure("EFORMAT", str(e)) from None
        except (OSError, RuntimeError) as e:
            raise Failure("EIO", str(e)) from None
        self.session_key = key
        self.log("info", msg="model loaded", path=path, dtype=self.o["dtype"],
                 pages=self.session.engine.num_pages, ctx_max=self.session.engine.ctx_max)
        return self.session

    def op_inspect(self, eff, body):
        """What a model file holds, without loading it (src/ops.c:204-276): @file, @layout (GGUF), @arch, one @kv per
        metadata key (for a folder: per config.json key), with --list-tensors one @tensor per tensor, @types per
        tensor type, @summary.  Needs no GPU."""
        import json
        import mmap
        from hfcpu_b200.config import known_architectures
        from hfcpu_b200.weights import gguf as G
        from hfcpu_b200.weights.safetensors_io import SafetensorsFile, WeightFormatError
        path = eff["model"]
        if not path:
            raise Failure("EINVAL", "inspect needs --model PATH")
        out, listing = self.out, eff["list_tensors"]
        known = set(known_architectures())

        def kv_event(key, kind, value):
            if isinstance(value, list):
                out.event("kv", key=key, type="array", elem=kind, count=len(value))
            elif isinstance(value, str) and len(value) > 160:
                out.event("kv", key=key, type=kind, value=value[:160], truncated_from=len(value))
            elif isinstance(value, float):
                out.event("kv", key=key, type=kind, value=f"{value:.9g}")
            else:
                out.event("kv", key=key, type=kind, value=value if isinstance(value, str) else json.dumps(value))

        tensors = []                                  # (name, type name, dims as stored, offset, bytes, supported)
        try:
            if os.path.isdir(path):
                cfg_path = os.path.join(path, "config.json")
                try:
                    with open(cfg_path) as f:
                        cfg = json.load(f)
                except (OSError, ValueError) as e:
                    raise Failure("EFORMAT", f"{cfg_path}: {e}") from None
                from hfcpu_b200.weights import find_weight_files
                for st_path in find_weight_files(path)[0]:           # the single file, or every shard
                    with SafetensorsFile(st_path) as st:
                        for name, (dt, shape, b, en) in st.entries.items():
                            tensors.append((name, str(dt).replace("torch.", ""), "x".join(map(str, shape)), b, en - b, True))
                        out.event("file", path=st_path, bytes=os.path.getsize(st_path), format="safetensors",
                                  tensors=len(st.entries), kv=len(cfg))
                arch = (cfg.get("architectures") or [cfg.get("model_type") or "(none)"])[0]
                for key, value in cfg.items():
                    kind = ("bool" if isinstance(value, bool) else "int" if isinstance(value, int) else
                            "float" if isinstance(value, float) else "string" if isinstance(value, str) else
                            "null" if value is None else "json")
                    kv_event(key, kind, value if kind != "json" or isinstance(value, list) else json.dumps(value))
            else:
                try:
                    f = open(path, "rb")
                except OSError as e:
                    raise Failure("EIO", f"{path}: {e.strerror}") from None
                with f:
                    size = os.fstat(f.fileno()).st_size
                    if size == 0:
                        raise WeightFormatError(f"{path}: empty file")
                    with mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as mm:
                        version, meta, kinds, infos, align, base = G.parse_gguf(mm, path)
                out.event("file", path=path, bytes=size, gguf_version=version, tensors=len(infos), kv=len(meta))
                out.event("layout", alignment=align, data_offset=base)
                arch = meta.get("general.architecture") or "(none)"
                for key, value in meta.items():
                    shown = (key.startswith("general.") or key.startswith(f"{arch}.") or isinstance(value, (list, str))
                             or key in ("tokenizer.ggml.model", "tokenizer.ggml.pre"))
                    if shown or listing:
                        kind = G.KV_TYPE_NAMES.get(kinds[key], str(kinds[key]))
                        kv_event(key, kind, bool(value) if kind == "bool" else value)
                for name, dims, tid, off in infos:
                    count = 1
                    for d in dims:
                        count *= d
                    esz = {0: 4, 1: 2, 30: 2}.get(tid)
                    tensors.append((name, G.TYPE_NAMES.get(tid, f"type{tid}"), "x".join(map(str, dims)), off,
                                    count * esz if esz else 0, esz is not None))
        except WeightFormatError as e:
            raise Failure("EFORMAT", str(e)) from None
        supported = arch in known
        out.event("arch", name=arch, supported="yes" if supported else "no",
                  **({} if supported else {"reason": "no model is registered under this name"}))
        by_type: Dict[str, list] = {}
        for name, tname, dims, off, nbytes, ok in tensors:
            if listing:
                out.event("tensor", name=name, type=tname, dims=dims, offset=off, bytes=nbytes)
            t = by_type.setdefault(tname, [0, 0, ok])
            t[0] += 1
            t[1] += nbytes
        for tname, (n, nbytes, ok) in by_type.items():
            out.event("types", name=tname, tensors=n, bytes=nbytes, supported="yes" if ok else "no")
        out.event("summary", tensor_bytes=sum(t[4] for t in tensors),
                  all_types_supported="yes" if all(t[5] for t in tensors) else "no")

    def op_generate(self, eff, body):
        from hfcpu_b200.engine import FinishEvent, Request, RequestError, TokenEvent
        from hfcpu_b200.sampling import SamplingParams
        self._reject_text(eff, body)
        sess = self._resident(eff)
        if eff["prompt_ids"] is None:
            raise Failure("EINVAL", "generate needs --prompt-ids (this engine has no tokenizer)")
        ids = parse_ids(eff["prompt_ids"], sess.model.plan.vocab_size)
        nseq = eff["n"]
        sch = sess.scheduler
        serial = self._serial
        reqs = []
        try:
            for i in range(nseq):
                p = SamplingParams(temp=eff["temp"], top_k=eff["top_k"], top_p=eff["top_p"], min_p=eff["min_p"],
                                   seed=(eff["seed"] + i) & ((1 << 64) - 1), max_tokens=eff["max_tokens"],
                                   logprobs=eff["logprobs"])
                # the cache of a request stays behind it, as the reference's one context does (src/ops.c:760-776)
                r = Request((serial, i), ids, p, eos_ids=sess.eos_ids, timeout=eff["timeout"], keep_cache=i == 0,
                            reuse_cache=eff["prefix_cache"])
                sch.submit(r)
                reqs.append(r)
        except RequestError as e:
            for r in reqs:
                sch.cancel(r.id)
            sch.run()
            raise Failure(e.code, str(e)) from None
        except ValueError as e:
            raise Failure("EINVAL", str(e)) from None
        self.out.event("prompt", tokens=len(ids), threads=0)
        t0 = time.perf_counter()
        t_prefill = None
        steps0 = sch.stats["steps"]
        prof = Profiler() if eff["profile"] else None
        self.cancel_requested = False
        errors = []
        while sch.has_work():
            if self.cancel_requested:
                for r in reqs:
                    sch.cancel(r.id)
                self.cancel_requested = False
            try:
                with (prof.phase("decode" if t_prefill is not None else "prefill") if prof else _null()):
                    events = sch.step()
            except Exception as e:
                # nothing of this request stays behind in the resident session
                sch.abort([r.id for r in reqs])
                sch.drop_retained()
                if prof:
                    prof.close()
                raise Failure(_code_of(e), str(e)) from None
            if t_prefill is None and all(r.computed >= len(r.prompt) or r.status == "finished" for r in reqs):
                t_prefill = time.perf_counter() - t0
                cached = sum(r.shared for r in reqs)
                self.out.event("prefill", tokens=len(ids), cached=reqs[0].shared, ms=f"{t_prefill * 1e3:.1f}",
                               tok_per_s=f"{(len(ids) * nseq - cached) / t_prefill if t_prefill > 0 else 0:.2f}",
                               kv_bytes=sess.engine.cache.bytes_in_use())
                if prof:
                    prof.emit(self.out, "prefill")
                t_dec0 = time.perf_counter()
            for ev in events:
                seq = {"seq": ev.req[1]} if nseq > 1 else {}
                if isinstance(ev, TokenEvent):
                    extra = {}
                    if ev.logprob is not None:
                        extra = {"logprob": f"{ev.logprob:.6f}", "top": " ".join(f"{i}:{lp:.6f}" for i, lp in ev.top)}
                    self.out.event("token", **seq, pos=ev.pos, id=ev.token, **extra)
                elif ev.error:
                    errors.append(ev.error)
        if prof:
            prof.emit(self.out, "decode")
            prof.close()
        if errors:
            code, _, msg = errors[0].partition(": ")
            raise Failure(code, msg)
        dt = time.perf_counter() - (t_dec0 if t_prefill is not None else t0)
        total = 0
        for r in reqs:
            seq = {"seq": r.id[1]} if nseq > 1 else {}
            total += len(r.generated)
            self.out.event("gen", **seq, tokens=len(r.generated), ms=f"{dt * 1e3:.1f}",
                           tok_per_s=f"{len(r.generated) / dt if dt > 0 else 0:.2f}", stop=r.stop)
        if nseq > 1:
            self.out.event("genall", sequences=nseq, tokens=total, ms=f"{dt * 1e3:.1f}",
                           tok_per_s=f"{total / dt if dt > 0 else 0:.2f}")

    def op_bench(self, eff, body):
        """Prefill and decode speed over synthetic ids (src/ops.c:942-1031): ids from xorshift modulo
        min(V, 2000) (src/ops.c:977-979), median over --probe-reps runs, one @bench line per batch size, with the
        fraction of the measured memory bandwidth the decode steps reach and of the tensor-core peak the prefill."""
        import statistics
        import torch
        from hfcpu_b200 import kernels
        from hfcpu_b200.cache import OutOfPages, OutOfSlots
        from hfcpu_b200.engine import StepEntry, measure
        sess = self._resident(eff)
        eng = sess.engine
        cuda = eng.device.type == "cuda"
        V = min(eng.model.plan.vocab_size, 2000)
        n_prompt, n_gen = eff["bench_prompt"], eff["bench_gen"]
        if n_prompt + n_gen > eng.ctx_max:
            raise Failure("ERANGE", f"--bench-prompt + --bench-gen exceed --ctx-max {eng.ctx_max}")
        try:
            batches = [int(x) for x in str(eff["bench_batch"]).replace(",", " ").split()]
        except ValueError:
            raise Failure("EINVAL", "--bench-batch must be a list of integers") from None
        peaks, peak_source = measure.load_peaks()
        chunk = sess.scheduler.prefill_chunk
        x = 0x9E3779B97F4A7C15
        sync = (lambda: torch.cuda.synchronize(eng.device)) if cuda else (lambda: None)
        for B in batches:
            if B < 1 or B > eng.max_requests:
                raise Failure("ERANGE", f"--bench-batch {B} exceeds --max-seqs {eng.max_requests}")
            pre, dec, pre_flops = [], [], 0.0
            ids_dev = [torch.empty(B, dtype=torch.int32, device=eng.device) for _ in range(2)]
            for _ in range(eff["probe_reps"]):
                prompts = []
                for b in range(B):
                    ids = []
                    for _ in range(n_prompt):
                        x ^= (x >> 12); x ^= (x << 25) & ((1 << 64) - 1); x ^= (x >> 27)
                        ids.append(((x * 0x2545F4914F6CDD1D) & ((1 << 64) - 1)) % V)
                    prompts.append(ids)
                    eng.add_request(("bench", b))
                try:
                    first = torch.empty(1, dtype=torch.int32, device=eng.device)
                    sync()
                    t0 = time.perf_counter()
                    pre_flops = 0.0
                    for b in range(B):
                        for a in range(0, n_prompt, chunk):
                            part = prompts[b][a:a + chunk]
                            last = a + len(part) == n_prompt
                            logits = eng.step([StepEntry(("bench", b), part, [len(part) - 1] if last else [])])
                            pre_flops += measure.step_flops(eng.model, [len(part)], [a + len(part)], 1 if last else 0)
                        kernels.argmax(logits, first)
                        ids_dev[0][b:b + 1].copy_(first)
                    sync()
                    pre.append(time.perf_counter() - t0)
                    entries = [StepEntry(("bench", b), [0], [0]) for b in range(B)]
                    t0 = time.perf_counter()
                    for i in range(n_gen):
                        # the ids the arg-max kernel wrote feed the next step on the device
                        logits = eng.step(entries, token_source=ids_dev[i & 1])
                        kernels.argmax(logits, ids_dev[(i + 1) & 1])
                    sync()
                    dec.append(time.perf_counter() - t0)
                    kernels.check_device_errors()
                except (OutOfPages, OutOfSlots) as e:
                    raise Failure("ENOMEM", str(e)) from None
                except Exception as e:
                    raise Failure(_code_of(e), str(e)) from None
                finally:
                    for b in range(B):
                        eng.finish_request(("bench", b))
            t_pre, t_dec = statistics.median(pre), statistics.median(dec)
            frac = measure.fractions(eng, decode_ms=t_dec / n_gen * 1e3, decode_kv_lens=[n_prompt + n_gen // 2] * B, peaks=peaks)
            mma = pre_flops / t_pre / (peaks["bf16_tflops"] * 1e12) if t_pre > 0 else 0.0
            self.out.event("bench", batch=B, prefill_tok_s=f"{B * n_prompt / t_pre:.2f}",
                           decode_tok_s=f"{B * n_gen / t_dec:.2f}", prompt_tokens=n_prompt, gen_tokens=n_gen,
                           hbm_frac=f"{frac.get('hbm_frac', 0.0):.4g}", mma_frac=f"{mma:.4g}", peaks=peak_source)


def _code_of(e: Exception) -> str:
    """The status name of an exception that ended a request."""
    from hfcpu_b200.cache import OutOfPages, OutOfSlots
    from hfcpu_b200.config import UnsupportedError
    if isinstance(e, (OutOfPages, OutOfSlots, MemoryError)):
        return "ENOMEM"
    if isinstance(e, UnsupportedError):
        return "ENOTSUP"
    if isinstance(e, (ValueError, KeyError)):
        return "EINVAL"
    return "EIO"


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class Profiler:
    """``--profile``: per stage (prefill, decode) the steps, their wall-clock time and where the device spent it, with
    the reference's phase names (src/model.h:75-79; its @profile line, src/ops.c:593-604): embed, glue (norms), qkv,
    attn, wo, gate_up, silu, down, head, quant, and ``sample``; ``host`` is the wall-clock time not covered by the
    phases.  While it is on, steps run kernel by kernel with CUDA events around each part's kernels, not as graphs."""

    def __init__(self):
        from hfcpu_b200 import kernels
        self.kernels = kernels
        self.acc: Dict[str, float] = {}
        self.steps: Dict[str, int] = {}
        kernels.profile.enable(True)

    def close(self):
        self.kernels.profile.enable(False)

    def phase(self, name):
        prof = self

        class P:
            def __enter__(self):
                self.t = time.perf_counter()

            def __exit__(self, *a):
                prof.acc[name] = prof.acc.get(name, 0.0) + time.perf_counter() - self.t
                prof.steps[name] = prof.steps.get(name, 0) + 1
                return False
        return P()

    def emit(self, out, stage):
        phases = self.kernels.profile.take()
        wall = self.acc.get(stage, 0.0) * 1e3
        out.event("profile", stage=stage, steps=self.steps.get(stage, 0), step_ms=f"{wall:.1f}",
                  **{k: f"{v:.1f}" for k, v in phases.items()}, host=f"{max(wall - sum(phases.values()), 0.0):.1f}")


def parse_ids(text: str, vocab: int) -> List[int]:
    """Token ids separated by spaces or commas, each below the vocabulary size (src/ops.c:563-589)."""
    out = []
    for w in text.replace(",", " ").split():
        try:
            v = int(w)
        except ValueError:
            raise Failure("EINVAL", f"'{w}' in the id list is not a token id") from None
        if not 0 <= v < vocab:
            raise Failure("EINVAL", f"token id {v} is outside the vocabulary of {vocab}")
        out.append(v)
    if not out:
        raise Failure("EINVAL", "empty prompt")
    return out


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--help" in argv or "-h" in argv:
        print(O.usage())
        return 0
    if "--version" in argv:
        import hfcpu_b200
        print(f"hfb200 {hfcpu_b200.__version__}")
        return 0
    try:
        cli = O.apply(O.defaults(), argv)
        base = O.load_settings(O.defaults(), cli["settings"]) if cli["settings"] else O.defaults()
        o = O.apply(base, argv)
    except O.OptionError as e:
        print(f"hfb200: {e}", file=sys.stderr)
        return 2
    out = EventWriter(sys.stdout.buffer)
    app = App(o, out)

    def on_int(sig, frame):
        if sig == signal.SIGINT and app.session is not None and app.session.scheduler.has_work():
            app.cancel_requested = True          # ends the running request with stop=cancel; the process stays
        else:
            app.interrupted = True
    signal.signal(signal.SIGINT, on_int)
    signal.signal(signal.SIGTERM, on_int)
    try:
        signal.signal(signal.SIGPIPE, signal.SIG_IGN)
    except (AttributeError, ValueError):
        pass
    for opt in O.OPTIONS:
        if opt.note == "ignored" and o[opt.key] != opt.default:
            app.log("info", msg="option accepted but has no effect in this engine", option=opt.name)

    mode = o["stdin_mode"]
    ok = True
    if mode == "none":
        ok = app.run_request(o, None)
    elif mode == "args":
        rd = RecordReader(0)
        while not app.interrupted and not out.err:
            got = rd.next(0x0A, int(o["max_record"]))
            if got is None:
                break
            status, rec = got
            if status:
                app.failed_request(status, f"request line rejected: line too long (limit --max-record {o['max_record']} bytes)")
                continue
            line = rec.decode("utf-8", "surrogateescape").rstrip("\r")
            if not line.strip() or line.startswith("#"):
                continue
            if line.startswith("!"):
                if line.startswith("!quit"):
                    break
                if line.startswith("!stats"):
                    extra = {}
                    if app.session is not None:
                        c = app.session.engine.cache
                        extra = {"pages_used": c.pages_in_use(), "pages_free": sum(c.free_pages()),
                                 "preemptions": app.session.scheduler.stats["preemptions"]}
                    out.event("stats", requests=app.n_requests, errors=app.n_errors, live_allocs=0, **extra)
                elif line.startswith("!cancel"):
                    out.event("info", msg="no request is running")
                else:
                    out.event("error", msg="unknown control line")
                continue
            try:
                eff = O.apply(o, O.shell_split(line), request_context=True)
            except O.OptionError as e:
                app.failed_request("EINVAL", str(e))
                continue
            app.run_request(eff, None)
    else:
        rd = RecordReader(0)
        sep = o["record_sep"]
        while not app.interrupted and not out.err:
            got = rd.next(sep, int(o["max_record"]))
            if got is None:
                break
            status, rec = got
            if status:
                app.failed_request(status, f"request rejected: record too large (limit --max-record {o['max_record']} bytes)")
            else:
                header, us, body = rec.partition(b"\x1f")
                if not us:
                    header, body = b"", rec
                try:
                    eff = O.apply(o, O.shell_split(header.decode("utf-8", "surrogateescape")), request_context=True)
                except O.OptionError as e:
                    app.failed_request("EINVAL", str(e))
                else:
                    app.run_request(eff, body)
            out.raw_byte(sep)
            out.flush()
    if app.interrupted:
        return 130
    if out.err:
        return 1
    return 0 if ok or mode != "none" else 1


if __name__ == "__main__":
    sys.exit(main())
