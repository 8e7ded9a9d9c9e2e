"""Table-driven options in the reference's vocabulary (src/opts.c:30-76).

One table serves the command line, the settings file and per-request option lines; the effective
options of a request are defaults < settings file < command line < per-request options
(docs/PROTOCOL.md:7-17).  Forms: ``--name value``, ``--name=value``, and for booleans ``--name``,
``--no-name``, ``--name=false`` (src/opts.c:272-311).  Sizes take K/M/G/T suffixes, 1024-based
(src/opts.c:142-166).  Session-only options are refused in a per-request line (src/opts.c:297-300).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

STR, INT, U64, SIZE, DBL, BOOL, ENUM, BYTE = "str", "int", "u64", "size", "dbl", "bool", "enum", "byte"
SESSION, REQUEST = "session", "request"


class OptionError(ValueError):
    pass


@dataclass(frozen=True)
class Opt:
    name: str
    kind: str
    scope: str
    default: Any
    help: str
    lo: Optional[float] = None
    hi: Optional[float] = None
    choices: Tuple[str, ...] = ()
    note: str = ""            # "text": needs a tokenizer, answered ENOTSUP; "ignored": parsed, has no effect here

    @property
    def key(self) -> str:
        return self.name.replace("-", "_")


OPTIONS: List[Opt] = [
    Opt("settings", STR, SESSION, None, "settings file (key = value lines)"),
    Opt("stdin-mode", ENUM, SESSION, "prompts", "prompts | args | none", choices=("prompts", "args", "none")),
    Opt("record-sep", BYTE, SESSION, 0x1E, "record separator byte (RS, US, LF, NUL, 0x1e, 30, or a char)"),
    Opt("control-fd", INT, SESSION, -1, "extra fd carrying control lines, -1 = none", -1, 1023, note="ignored"),
    Opt("cache-dir", STR, SESSION, None, "directory for profiles and persistent caches", note="ignored"),
    Opt("cache-quota", SIZE, SESSION, 0, "persistent cache size limit, 0 = disabled", note="ignored"),
    Opt("cache-min-free", SIZE, SESSION, 10 << 30, "free space always left on the cache filesystem", note="ignored"),
    Opt("threads", INT, SESSION, 0, "worker threads, 0 = auto (the GPU engine has none)", 0, 256, note="ignored"),
    Opt("ctx-init", SIZE, SESSION, 2048, "initial context tokens", note="ignored"),
    Opt("ctx-step", SIZE, SESSION, 1024, "context growth increment in tokens", note="ignored"),
    Opt("ctx-max", SIZE, SESSION, 32768, "maximum context tokens"),
    Opt("max-record", SIZE, SESSION, 64 << 20, "largest accepted prompt or request line"),
    Opt("batch", INT, SESSION, 0, "prefill tokens per step at most, 0 = as many as --max-batched-tokens allows (the "
        "reference's default of 64 is a CPU's step; here a step of 64 tokens costs a prompt seven times the time)", 0, 4096),
    Opt("log-level", ENUM, SESSION, "info", "error | warn | info | debug", choices=("error", "warn", "info", "debug")),
    # engine options (no counterpart in the reference)
    Opt("dtype", ENUM, SESSION, "bf16", "bf16 | fp32 (fp32 = the whole model in true 32-bit)",
        choices=("bf16", "fp32", "bfloat16", "float32")),
    Opt("kv-block", INT, SESSION, 16, "tokens per cache page", 1, 1024),
    Opt("kv-pages", SIZE, SESSION, 0, "cache pages per layer group, 0 = from --kv-mem or free memory"),
    Opt("kv-mem", SIZE, SESSION, 0, "bytes for the cache, 0 = most of the free memory"),
    Opt("max-seqs", INT, SESSION, 64, "requests decoded together at most", 1, 4096),
    Opt("max-batched-tokens", INT, SESSION, 2048, "tokens per step at most", 1, 1 << 20),
    Opt("eos-ids", STR, SESSION, None, "end-of-generation token ids, space or comma separated (default: config.json)"),
    Opt("random-weights", STR, SESSION, None, "a config.json: run a model of that configuration with seeded random "
        "weights made on the device (no --model needed)"),
    Opt("weights-seed", U64, SESSION, None, "seed of --random-weights (default: the command line's --seed)"),
    Opt("weights-std", DBL, SESSION, 0.02, "standard deviation of --random-weights", 0, 10),

    Opt("op", STR, REQUEST, "generate", "generate | bench | echo"),
    Opt("model", STR, REQUEST, None, "model folder (config.json + safetensors, one file or shards) or a .gguf file"),
    Opt("id", STR, REQUEST, None, "request id echoed in the response"),
    Opt("chat", ENUM, REQUEST, None, "raw | auto | chatml | llama3", choices=("raw", "auto", "chatml", "llama3"), note="text"),
    Opt("system", STR, REQUEST, None, "system prompt text", note="text"),
    Opt("system-file", STR, REQUEST, None, "system prompt from a file", note="text"),
    Opt("prompt", STR, REQUEST, None, "prompt text (short prompts)", note="text"),
    Opt("prompt-file", STR, REQUEST, None, "prompt from a file", note="text"),
    Opt("prompt-ids", STR, REQUEST, None, "prompt as token ids, space or comma separated"),
    Opt("n", INT, REQUEST, 1, "generate: completions decoded together from one prompt (seeds seed, seed+1, ...)", 1, 64),
    Opt("temp", DBL, REQUEST, 0.8, "sampling temperature", 0, 5),
    Opt("top-k", INT, REQUEST, 40, "top-k, 0 = off", 0, 1000000),
    Opt("top-p", DBL, REQUEST, 0.95, "top-p", 0, 1),
    Opt("min-p", DBL, REQUEST, 0.05, "min-p", 0, 1),
    Opt("seed", U64, REQUEST, 0, "RNG seed (deterministic)"),
    Opt("max-tokens", INT, REQUEST, 512, "maximum new tokens", 1, 1 << 24),
    Opt("logprobs", INT, REQUEST, 0, "top-N logprobs per token, 0 = off", 0, 100),
    Opt("stop", STR, REQUEST, None, "generate: stop before this text", note="text"),
    Opt("stop-on-repeat", BOOL, REQUEST, True, "stop on repetition loops", note="ignored"),
    Opt("timeout", DBL, REQUEST, 0.0, "per-request time limit in seconds, 0 = none", 0, 1e7),
    Opt("profile", BOOL, REQUEST, False, "generate: report per-phase time of prefill and decode (@profile events)"),
    Opt("list-tensors", BOOL, REQUEST, False, "inspect: list every tensor"),
    Opt("prefix-cache", BOOL, REQUEST, True, "generate: start on the cache pages of the previous request's tokens where "
        "the prompt begins with the same ones (default on)"),
    Opt("parse-special", BOOL, REQUEST, True, "tokenize: recognise special tokens in the text", note="text"),
    Opt("bench-prompt", INT, REQUEST, 256, "bench: prompt tokens to prefill", 1, 32768),
    Opt("bench-gen", INT, REQUEST, 32, "bench: tokens to decode", 1, 4096),
    Opt("bench-batch", STR, REQUEST, "1", "bench: batch sizes to try, e.g. 1,8,64"),
    Opt("probe-reps", INT, REQUEST, 1, "bench: repeat N times, report the median", 1, 32),
]
BY_NAME: Dict[str, Opt] = {o.name: o for o in OPTIONS}


def defaults() -> Dict[str, Any]:
    return {o.key: o.default for o in OPTIONS}


def parse_size(text: str) -> int:
    t = text.strip()
    mult = 1
    if t and t[-1] in "kKmMgGtT":
        mult = 1024 ** ("kmgt".index(t[-1].lower()) + 1)
        t = t[:-1]
    try:
        v = int(t, 0)
    except ValueError:
        raise OptionError(f"'{text}' is not a size") from None
    if v < 0:
        raise OptionError(f"'{text}' is negative")
    return v * mult


def parse_byte(text: str) -> int:
    names = {"RS": 0x1E, "US": 0x1F, "LF": 0x0A, "NUL": 0}
    if text in names:
        return names[text]
    if len(text) == 1 and not text.isdigit():
        return ord(text)
    try:
        v = int(text, 0)
    except ValueError:
        raise OptionError(f"'{text}' is not a byte") from None
    if not 0 <= v <= 255:
        raise OptionError(f"'{text}' is not a byte")
    return v


def _convert(o: Opt, text: str) -> Any:
    try:
        if o.kind == STR:
            return text
        if o.kind == INT:
            v = int(text, 0)
        elif o.kind == U64:
            v = int(text, 0)
            if not 0 <= v < 1 << 64:
                raise ValueError
        elif o.kind == SIZE:
            return parse_size(text)
        elif o.kind == DBL:
            v = float(text)
        elif o.kind == BOOL:
            if text.lower() in ("1", "true", "yes", "on"):
                return True
            if text.lower() in ("0", "false", "no", "off"):
                return False
            raise ValueError
        elif o.kind == ENUM:
            if text not in o.choices:
                raise OptionError(f"--{o.name}: '{text}' is not one of {' | '.join(o.choices)}")
            return text
        elif o.kind == BYTE:
            return parse_byte(text)
    except ValueError:
        raise OptionError(f"--{o.name}: '{text}' is not a valid value") from None
    if o.lo is not None and v < o.lo or o.hi is not None and v > o.hi:
        raise OptionError(f"--{o.name}: {text} is outside [{o.lo:g}, {o.hi:g}]")
    return v


def apply(opts: Dict[str, Any], argv: List[str], request_context: bool = False) -> Dict[str, Any]:
    """Apply ``argv`` on top of ``opts`` (a copy is returned)."""
    out = copy.copy(opts)
    i = 0
    while i < len(argv):
        a = argv[i]
        i += 1
        if not a.startswith("--") or len(a) < 3:
            raise OptionError(f"unexpected argument '{a}'")
        name, eq, val = a[2:].partition("=")
        negate = False
        if name not in BY_NAME and name.startswith("no-") and name[3:] in BY_NAME and BY_NAME[name[3:]].kind == BOOL:
            name, negate = name[3:], True
        if name not in BY_NAME:
            raise OptionError(f"unknown option '--{name}'")
        o = BY_NAME[name]
        if request_context and o.scope == SESSION:
            raise OptionError(f"--{name} can only be set at startup")
        if o.kind == BOOL:
            if negate:
                if eq:
                    raise OptionError(f"--no-{name} takes no value")
                out[o.key] = False
            else:
                out[o.key] = _convert(o, val) if eq else True
            continue
        if not eq:
            if i >= len(argv):
                raise OptionError(f"--{name} needs a value")
            val = argv[i]
            i += 1
        out[o.key] = _convert(o, val)
    return out


def load_settings(opts: Dict[str, Any], path: str) -> Dict[str, Any]:
    """``key = value`` lines, ``#`` comments (src/opts.c:313-358)."""
    out = copy.copy(opts)
    try:
        lines = open(path).read().splitlines()
    except OSError as e:
        raise OptionError(f"cannot read settings file {path}: {e.strerror}") from None
    for n, line in enumerate(lines, 1):
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        key, eq, val = line.partition("=")
        if not eq:
            raise OptionError(f"{path}:{n}: expected key = value")
        try:
            out = apply(out, [f"--{key.strip()}={val.strip()}"])
        except OptionError as e:
            raise OptionError(f"{path}:{n}: {e}") from None
    return out


def shell_split(line: str) -> List[str]:
    """POSIX-shell word splitting without expansion (src/opts.c:372-442): single quotes are literal; double
    quotes allow \\" \\\\ \\n \\t; outside quotes a backslash escapes the next character."""
    words, cur, have = [], [], False
    i, n = 0, len(line)
    while i < n:
        c = line[i]
        if c in " \t\r\n":
            if have:
                words.append("".join(cur))
                cur, have = [], False
            i += 1
        elif c == "'":
            j = line.find("'", i + 1)
            if j < 0:
                raise OptionError("unterminated single quote")
            cur.append(line[i + 1:j])
            have = True
            i = j + 1
        elif c == '"':
            i += 1
            while True:
                if i >= n:
                    raise OptionError("unterminated double quote")
                c = line[i]
                if c == '"':
                    break
                if c == "\\" and i + 1 < n and line[i + 1] in '"\\nt':
                    cur.append({"n": "\n", "t": "\t"}.get(line[i + 1], line[i + 1]))
                    i += 2
                else:
                    cur.append(c)
                    i += 1
            have = True
            i += 1
        elif c == "\\":
            if i + 1 >= n:
                raise OptionError("trailing backslash")
            cur.append(line[i + 1])
            have = True
            i += 2
        else:
            cur.append(c)
            have = True
            i += 1
    if have:
        words.append("".join(cur))
    return words


def usage() -> str:
    lines = ["usage: hfb200 [options]   (requests on stdin, events on stdout; see --stdin-mode)", ""]
    for scope, title in ((SESSION, "startup only"), (REQUEST, "per request")):
        lines.append(f"{title}:")
        for o in OPTIONS:
            if o.scope == scope:
                extra = {"text": " [needs a tokenizer: ENOTSUP]", "ignored": " [accepted, no effect]"}.get(o.note, "")
                lines.append(f"  --{o.name:<20} {o.help}{extra}")
        lines.append("")
    return "\n".join(lines)
