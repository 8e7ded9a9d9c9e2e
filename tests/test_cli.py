"""Options, protocol and the command line (what the reference covers in tests/test_opts.c and tests/e2e.pl)."""
import io
import os
import subprocess
import sys

import pytest

import plain_qwen2 as plain
from conftest import ROOT, make_requests


def test_option_forms_and_ranges():
    from hfcpu_b200.cli import opts as O
    d = O.defaults()
    assert d["temp"] == 0.8 and d["top_k"] == 40 and d["top_p"] == 0.95 and d["min_p"] == 0.05
    assert d["max_tokens"] == 512 and d["batch"] == 0 and d["ctx_max"] == 32768 and d["record_sep"] == 0x1E
    o = O.apply(d, ["--temp", "0.5", "--top-k=7", "--no-profile", "--profile", "--ctx-max", "4K", "--record-sep", "US"])
    assert o["temp"] == 0.5 and o["top_k"] == 7 and o["profile"] is True and o["ctx_max"] == 4096 and o["record_sep"] == 0x1F
    assert O.apply(d, ["--profile=false"])["profile"] is False
    assert d["temp"] == 0.8                                   # the input is not modified
    for bad in (["--temp", "9"], ["--top-k", "-1"], ["--nope"], ["--temp"], ["stray"], ["--stdin-mode", "x"],
                ["--no-temp"], ["--n", "65"]):
        with pytest.raises(O.OptionError):
            O.apply(d, bad)
    with pytest.raises(O.OptionError):                        # session-only options are refused per request
        O.apply(d, ["--ctx-max", "100"], request_context=True)
    assert O.parse_size("2M") == 2 << 20 and O.parse_size("0x10") == 16


def test_shell_split():
    from hfcpu_b200.cli.opts import OptionError, shell_split
    assert shell_split("--id 'a b' --x \"q\\\"r\\n\" c\\ d") == ["--id", "a b", "--x", 'q"r\n', "c d"]
    assert shell_split("  ") == [] and shell_split("''") == [""]
    for bad in ("'open", '"open', "trail\\"):
        with pytest.raises(OptionError):
            shell_split(bad)


def test_settings_file(tmp_path):
    from hfcpu_b200.cli import opts as O
    p = tmp_path / "s.conf"
    p.write_text("# comment\ntemp = 0.25\nbatch=128\n")
    o = O.load_settings(O.defaults(), str(p))
    assert o["temp"] == 0.25 and o["batch"] == 128
    p.write_text("bogus = 1\n")
    with pytest.raises(O.OptionError):
        O.load_settings(O.defaults(), str(p))


def test_event_quoting():
    from hfcpu_b200.cli.proto import EventWriter, quote
    assert quote("abc") == "abc" and quote("") == '""' and quote("a b") == '"a b"' and quote("a=b") == '"a=b"'
    assert quote('q"\\\n\t\x01') == '"q\\"\\\\\\n\\t\\x01"'
    f = io.BytesIO()
    w = EventWriter(f)
    w.event("token", pos=3, id=17)
    w.payload("prompt", b"hi there")
    assert f.getvalue() == b"@token pos=3 id=17\n@prompt len=8\nhi there\n"


def test_record_reader_resyncs_after_an_oversize_record():
    from hfcpu_b200.cli.proto import RecordReader
    r, w = os.pipe()
    os.write(w, b"one\x1e" + b"x" * 5000 + b"\x1etwo\x1etail")
    os.close(w)
    rd = RecordReader(r)
    got = []
    while True:
        x = rd.next(0x1E, 100)
        if x is None:
            break
        got.append(x)
    assert got == [(None, b"one"), ("ERANGE", b""), (None, b"two"), (None, b"tail")]


def _run_cli(args, stdin=b""):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, os.path.join(ROOT, "tests")]))
    code = ("import sys; from hfcpu_b200 import kernels; from emu_backend import EmuBackend; "
            "kernels.set_backend(EmuBackend()); import hfcpu_b200.api as api; "
            "orig = api.Session.__init__\n"
            "def init(self, model, **kw):\n    kw['device'] = 'cpu'; orig(self, model, **kw)\n"
            "api.Session.__init__ = init\n"
            "import hfcpu_b200.cli.main as cm; cm.App.device = 'cpu'\n"
            "from hfcpu_b200.cli.main import main; sys.exit(main(sys.argv[1:]))")
    return subprocess.run([sys.executable, "-c", code, *args], input=stdin, capture_output=True, env=env, timeout=120)


def test_generate_events_and_errors(tiny_folders):
    folder = tiny_folders["A"]
    prompt = make_requests("A", [12], seed=3)["r0"]
    ids = " ".join(map(str, prompt))
    common = ["--dtype", "fp32", "--kv-pages", "32", "--ctx-max", "256", "--model", folder]
    r = _run_cli(["--stdin-mode", "none", "--op", "generate", "--prompt-ids", ids, "--temp", "0", "--max-tokens", "5",
                  "--logprobs", "3", *common])
    assert r.returncode == 0, r.stderr.decode()
    lines = r.stdout.decode().splitlines()
    assert lines[0].startswith("@begin id=1 op=generate") and lines[-1].startswith("@done status=ok")
    assert lines[1] == "@prompt tokens=12 threads=0" and lines[2].startswith("@prefill tokens=12 cached=0 ")
    toks = [l for l in lines if l.startswith("@token")]
    cfg, W = plain.read_folder(folder)
    want = plain.greedy(cfg, W, prompt, 5)
    assert [int(l.split("id=")[1].split()[0]) for l in toks] == want
    assert all("logprob=" in l and "top=" in l for l in toks)
    assert [l for l in lines if l.startswith("@gen ")][0].endswith("stop=length")
    # args mode: several requests to one resident model, errors answered per request, controls
    script = (f"--op generate --prompt-ids '{ids}' --temp 0 --max-tokens 2 --id a\n"
              f"--op generate --prompt 'some text' --id b\n"
              f"--op generate --prompt-ids '1 2 9999' --id c\n"
              f"--op generate --prompt-ids '{ids}' --n 2 --temp 0.7 --seed 4 --max-tokens 3 --id d\n"
              f"--ctx-max 5\n!stats\n!quit\n--op echo\n").encode()
    r = _run_cli(["--stdin-mode", "args", *common], script)
    out = r.stdout.decode()
    assert r.returncode == 0, r.stderr.decode()
    assert "@done status=error code=ENOTSUP" in out and "@done status=error code=EINVAL" in out
    assert out.count("@begin") == 5 and "@genall sequences=2 tokens=6" in out and "seq=1" in out
    assert "@stats requests=5 errors=3" in out and "op=echo" not in out
    assert r.stderr.decode().count("model loaded") == 1          # the model stays resident between requests


def test_the_next_request_starts_on_the_previous_requests_cache(tiny_folders):
    """--prefix-cache (on by default, src/opts.c:100): a prompt that begins like the previous request's tokens
    reports them as cached (src/ops.c:771-776, :802) and generates what it generates without them."""
    folder = tiny_folders["A"]
    first = make_requests("A", [21], seed=6)["r0"]
    cfg, W = plain.read_folder(folder)
    said = plain.greedy(cfg, W, first, 4)
    follow = first + said + make_requests("A", [6], seed=7)["r0"]
    want = plain.greedy(cfg, W, follow, 3)
    f, g = " ".join(map(str, first)), " ".join(map(str, follow))
    common = ["--dtype", "fp32", "--kv-pages", "40", "--kv-block", "4", "--ctx-max", "256", "--model", folder]
    for flag, cached in (("", (21 + 4 - 1) // 4 * 4), ("--no-prefix-cache", 0)):
        script = (f"--op generate --prompt-ids '{f}' --temp 0 --max-tokens 4 --id a\n"
                  f"--op generate --prompt-ids '{g}' --temp 0 --max-tokens 3 --id b {flag}\n").encode()
        r = _run_cli(["--stdin-mode", "args", *common], script)
        assert r.returncode == 0, r.stderr.decode()
        lines = r.stdout.decode().splitlines()
        prefills = [l for l in lines if l.startswith("@prefill")]
        assert len(prefills) == 2, r.stdout.decode() + r.stderr.decode()
        assert prefills[0].startswith("@prefill tokens=21 cached=0 ")
        assert prefills[1].startswith(f"@prefill tokens={len(follow)} cached={cached} "), prefills[1]
        toks = [int(l.split("id=")[1].split()[0]) for l in lines if l.startswith("@token")]
        assert toks == said + want


def test_startup_errors_exit_2():
    r = _run_cli(["--temp", "77"])
    assert r.returncode == 2 and b"--temp" in r.stderr


def test_inspect_lists_what_a_model_file_holds(tiny_folders, tmp_path):
    """--op inspect (src/ops.c:204-276) on a model folder and on a GGUF file, without loading either."""
    import torch
    import hfcpu_b200
    from hfcpu_b200.weights import gguf
    folder = tiny_folders["A"]
    r = _run_cli(["--stdin-mode", "none", "--op", "inspect", "--model", folder, "--list-tensors"])
    assert r.returncode == 0, r.stderr.decode()
    lines = r.stdout.decode().splitlines()
    assert lines[1].startswith("@file path=") and "format=safetensors" in lines[1]
    assert any(l.startswith("@arch name=Qwen2ForCausalLM supported=yes") for l in lines)
    assert any(l.startswith("@kv key=hidden_size type=int value=") for l in lines)
    tensors = [l for l in lines if l.startswith("@tensor ")]
    assert any("name=model.embed_tokens.weight type=float32 dims=" in l for l in tensors)
    summary = [l for l in lines if l.startswith("@summary")][0]
    assert "all_types_supported=yes" in summary
    total = sum(int(l.split("bytes=")[1].split()[0]) for l in tensors)
    assert f"tensor_bytes={total}" in summary and lines[-1].startswith("@done status=ok")
    # the same model as a GGUF file
    model = hfcpu_b200.load_model(folder, torch.float32, "cpu")
    path = str(tmp_path / "tiny.gguf")
    import json, os
    cfg = json.load(open(os.path.join(folder, "config.json")))
    from hfcpu_b200.weights.safetensors_io import SafetensorsFile
    with SafetensorsFile(os.path.join(folder, "model.safetensors")) as st:
        gguf.write_gguf(path, cfg, {n: st.tensor(n) for n in st.names()})
    r = _run_cli(["--stdin-mode", "none", "--op", "inspect", "--model", path])
    assert r.returncode == 0, r.stderr.decode()
    out = r.stdout.decode()
    assert "@file path=" in out and "gguf_version=3" in out and "@layout alignment=32" in out
    assert "@arch name=qwen2 supported=yes" in out and "@kv key=qwen2.block_count type=u32 value=" in out
    # (the folder stores the tied head beside the embedding; the GGUF file, like the reference's, leaves it out)
    head = sum(int(l.split("bytes=")[1].split()[0]) for l in tensors if "name=lm_head.weight " in l)
    assert "@types name=F32 tensors=" in out and "@tensor " not in out and f"tensor_bytes={total - head}" in out
    # not a model file
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUX" + b"\0" * 40)
    r = _run_cli(["--stdin-mode", "none", "--op", "inspect", "--model", str(bad)])
    assert "@done status=error code=EFORMAT" in r.stdout.decode()
    r = _run_cli(["--stdin-mode", "none", "--op", "inspect"])
    assert "code=EINVAL" in r.stdout.decode() and "inspect needs --model" in r.stdout.decode()


def _golden_folder(tmp_path, name):
    """The model of tests/golden/tiny_<name>.json as a folder (float32, window off, as the reference ran it)."""
    import json
    import torch
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.weights import weights_path, write_safetensors
    from test_golden import _weights
    record = json.load(open(os.path.join(ROOT, "tests", "golden", f"tiny_{name}.json")))
    folder = str(tmp_path / f"golden_{name}")
    config_from_dict(record["config"]).save(folder)
    write_safetensors(weights_path(folder), _weights(record))
    return record, folder


@pytest.mark.parametrize("name", ["A", "B"])
def test_logprob_values_are_the_references(tmp_path, name):
    """--logprobs 5 on the models the reference ran (tests/golden): the same token ids, the same five candidates, and
    log-probabilities within the bound its own oracle uses for float weights (4e-3; its cache is float16,
    src/model.c:599-600).  Formula: src/sample.c:25-55."""
    record, folder = _golden_folder(tmp_path, name)
    worst = 0.0
    for case in record["cases"]:
        r = _run_cli(["--stdin-mode", "none", "--op", "generate", "--model", folder, "--dtype", "fp32", "--kv-pages", "64",
                      "--kv-block", "8", "--ctx-max", "256", "--prompt-ids", " ".join(map(str, case["prompt"])),
                      "--temp", "0", "--max-tokens", str(len(case["tokens"])), "--logprobs", "5"])
        assert r.returncode == 0, r.stderr.decode()
        toks = [l for l in r.stdout.decode().splitlines() if l.startswith("@token")]
        assert len(toks) == len(case["tokens"])
        for line, want in zip(toks, case["tokens"]):
            f = dict(kv.split("=", 1) for kv in line.replace('top="', "top=").rstrip('"').split(" ", 4)[1:])
            top = [(int(a.split(":")[0]), float(a.split(":")[1])) for a in f["top"].split()]
            assert int(f["id"]) == want["id"] and top[0][0] == want["id"]
            worst = max(worst, abs(float(f["logprob"]) - want["logprob"]))
            theirs = dict((i, v) for i, v in want["top"])
            for i, v in top:
                if i in theirs:
                    worst = max(worst, abs(v - theirs[i]))
                else:                                  # fifth and sixth candidate closer than the bound
                    assert abs(v - want["top"][-1][1]) < 8e-3
    assert worst < 4e-3, worst


def test_bench_random_weights_and_profile(tmp_path):
    """--random-weights CONFIG.json (the role of tools/mkmodel.pl:104-119) serves --op generate and --op bench without a
    model file; @bench carries the fractions beside the reference's fields (src/ops.c:1023); --profile splits a
    stage into the reference's phases (src/ops.c:593-604)."""
    import json
    import torch
    from conftest import TINY_A
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(TINY_A))
    common = ["--dtype", "fp32", "--kv-pages", "64", "--ctx-max", "256", "--random-weights", str(cfg_path),
              "--weights-seed", "5", "--weights-std", "0.2"]
    prompt = make_requests("A", [9], seed=4)["r0"]
    script = (f"--op generate --prompt-ids '{' '.join(map(str, prompt))}' --temp 0 --max-tokens 4 --profile\n"
              "--op bench --bench-prompt 24 --bench-gen 6 --bench-batch 1,3 --probe-reps 2\n").encode()
    r = _run_cli(["--stdin-mode", "args", *common], script)
    assert r.returncode == 0, r.stderr.decode()
    lines = r.stdout.decode().splitlines()
    W = random_tensors(build_model_specs(config_from_dict(TINY_A)), 5, torch.float32, std=0.2)
    toks = [int(l.split("id=")[1].split()[0]) for l in lines if l.startswith("@token")]
    assert toks == plain.greedy(TINY_A, W, prompt, 4)
    prof = [l for l in lines if l.startswith("@profile")]
    assert [l.split()[1] for l in prof] == ["stage=prefill", "stage=decode"]
    for key in ("steps=", "step_ms=", "embed=", "glue=", "qkv=", "attn=", "wo=", "gate_up=", "silu=", "down=", "head=",
                "quant=", "sample=", "host="):
        assert key in prof[1], key
    bench = [l for l in lines if l.startswith("@bench")]
    assert len(bench) == 2 and bench[0].startswith("@bench batch=1 prefill_tok_s=") and "batch=3" in bench[1]
    for l in bench:
        f = dict(kv.split("=", 1) for kv in l.split()[1:])
        assert f["prompt_tokens"] == "24" and f["gen_tokens"] == "6" and float(f["decode_tok_s"]) > 0
        assert 0 < float(f["hbm_frac"]) < 1 and 0 < float(f["mma_frac"]) < 1 and f["peaks"] in ("measured", "fallback")
    assert r.stderr.decode().count("model loaded") == 1
    # a bench that cannot fit answers ERANGE / ENOMEM and leaves the session usable
    script = ("--op bench --bench-prompt 250 --bench-gen 10\n--op bench --bench-prompt 200 --bench-gen 8 --bench-batch 2\n"
              "--op bench --bench-prompt 8 --bench-gen 2\n").encode()
    r = _run_cli(["--stdin-mode", "args", *common, "--kv-pages", "16"], script)
    out = r.stdout.decode()
    assert "code=ERANGE" in out and "code=ENOMEM" in out and out.count("@bench batch=1") == 1, out


def test_interrupt_cancels_the_running_request_and_the_process_stays(tiny_folders):
    """SIGINT while a request generates ends it with stop=cancel; the process stays and serves the next request
    (src/main.c:20-27, src/ops.c:829-833)."""
    import signal
    import time
    folder = tiny_folders["A"]
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, os.path.join(ROOT, "tests")]))
    code = ("import sys; from hfcpu_b200 import kernels; from emu_backend import EmuBackend; "
            "kernels.set_backend(EmuBackend()); import hfcpu_b200.api as api; "
            "orig = api.Session.__init__\n"
            "def init(self, model, **kw):\n    kw['device'] = 'cpu'; orig(self, model, **kw)\n"
            "api.Session.__init__ = init\n"
            "from hfcpu_b200.cli.main import main; sys.exit(main(sys.argv[1:]))")
    p = subprocess.Popen([sys.executable, "-c", code, "--stdin-mode", "args", "--dtype", "fp32", "--kv-pages", "64",
                          "--ctx-max", "256", "--model", folder], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, env=env)
    try:
        p.stdin.write(b"--op generate --prompt-ids '1 2 3' --temp 0 --max-tokens 200 --id long\n")
        p.stdin.flush()
        lines = []
        while True:
            line = p.stdout.readline().decode()
            assert line, p.stderr.read().decode()
            lines.append(line)
            if line.startswith("@token"):
                break
        p.send_signal(signal.SIGINT)
        while not lines[-1].startswith("@done"):
            line = p.stdout.readline().decode()
            assert line
            lines.append(line)
        gen = [l for l in lines if l.startswith("@gen ")][0]
        assert gen.strip().endswith("stop=cancel") and lines[-1].startswith("@done status=ok")
        assert 1 <= int(gen.split("tokens=")[1].split()[0]) < 200
        p.stdin.write(b"--op generate --prompt-ids '4 5' --temp 0 --max-tokens 2 --id next\n!stats\n!quit\n")
        p.stdin.flush()
        out, _ = p.communicate(timeout=60)
        out = out.decode()
        assert "@begin id=next" in out and out.count("@token") == 2 and "stop=length" in out
        assert "pages_used=" in out and p.returncode == 0
    finally:
        if p.poll() is None:
            p.kill()
