#!/usr/bin/env python3
"""Makes tests/golden/*.json: what the reference's own C code computes on tiny random models.

    python tests/golden/make_golden.py /path/to/ebowh-hf.cpu

The reference tree is copied to a temporary folder and built there with its own Makefile (plain C99,
no dependencies).  For each tiny configuration this script writes random float32 weights as one of
the reference's GGUF files (through the engine's exporter) and runs

    hfcpu --stdin-mode none --op generate --model M.gguf --prompt-ids "..." --temp 0 --max-tokens N --logprobs 5

recording the greedy tokens with their log-probabilities and top-5 candidates (src/ops.c:846-865).
tests/test_golden.py compares the plain implementation with these records.  The reference has no
sliding window, so the windowed configuration is exported with the window switched off; its
float16 key/value cache (src/model.c:599-600) bounds the agreement at about 1e-3 in log-probability
(its own oracle accepts 4e-3, tests/oracle.pl:18-23).

Further records:

* ``tiny_A_rope8.json``: configuration A with ``qwen2.rope.dimension_count = 8`` (half of its head size;
  src/model.c:132-133), greedy as above.
* ``"sampled"`` in ``tiny_A.json`` / ``tiny_B.json``: the same models run with ``--temp/--top-k/--top-p/--min-p/--seed``
  and with ``--n 3`` (sequence i draws with seed + i, src/ops.c:819); tokens per sequence.  These runs keep a
  dozen candidates at most: the reference's logits carry the rounding of its float16 cache, and a draw among
  hundreds of candidates of equal weight would fall on a neighbour every few tokens (the sampler over the whole
  vocabulary is pinned by ``sampler.json``, on exact logits).
* ``sampler.json``: the reference's sampler alone, through a small C harness (below) that is linked with the
  reference's own ``src/sample.o`` and ``src/mathx.o`` and calls ``hfc_rng_seed`` / ``hfc_rng_uniform`` /
  ``hfc_sample`` (src/sample.h): the first draws of the generator for a few seeds, and the tokens it picks from
  rows of synthetic logits (``sampler_logits`` in tests/conftest.py makes the same rows from integer arithmetic)
  under several settings, several draws in a row from one generator.
"""
import json
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.dirname(os.path.dirname(HERE)), os.path.dirname(HERE)]

import torch  # noqa: E402

from conftest import TINY, make_requests  # noqa: E402


HARNESS = r"""
#include <stdio.h>
#include <stdlib.h>
#include "sample.h"
/* stdin: "rng SEED N" -> N uniforms as %.9g; "pick SEED TEMP TOPK TOPP MINP ROW DRAWS" -> DRAWS tokens from row ROW */
int main(int argc, char **argv)
{
    size_t V = (size_t)atol(argv[2]), rows = (size_t)atol(argv[3]);
    float *L = malloc(V * rows * sizeof(float));
    FILE *f = fopen(argv[1], "rb");
    char op[8];
    if (argc < 4 || !f || fread(L, sizeof(float), V * rows, f) != V * rows) return 2;
    while (scanf("%7s", op) == 1) {
        unsigned long long seed; int n, i; hfc_rng r;
        if (op[0] == 'r') {
            if (scanf("%llu %d", &seed, &n) != 2) return 3;
            hfc_rng_seed(&r, seed);
            for (i = 0; i < n; i++) printf("%.9g ", hfc_rng_uniform(&r));
        } else {
            hfc_sampler p; int row; uint32_t tok;
            if (scanf("%llu %f %d %f %f %d %d", &seed, &p.temp, &p.top_k, &p.top_p, &p.min_p, &row, &n) != 7) return 3;
            hfc_rng_seed(&r, seed);
            for (i = 0; i < n; i++) { if (hfc_sample(L + (size_t)row * V, V, &p, &r, &tok)) return 4; printf("%u ", tok); }
        }
        printf("\n");
    }
    return 0;
}
"""

SAMPLED_RUNS = [
    {"temp": 0.8, "top_k": 40, "top_p": 0.95, "min_p": 0.05, "seed": 5, "n": 1},
    {"temp": 1.3, "top_k": 12, "top_p": 0.7, "min_p": 0.0, "seed": 9, "n": 1},
    {"temp": 1.0, "top_k": 8, "top_p": 1.0, "min_p": 0.0, "seed": 2, "n": 3},
]
SAMPLER_SETTINGS = [
    (0.8, 40, 0.95, 0.05), (1.3, 0, 0.7, 0.0), (1.0, 0, 1.0, 0.0), (0.5, 5, 1.0, 0.0), (2.0, 0, 1.0, 0.2),
    (0.0, 40, 0.95, 0.05), (1.0, 1, 1.0, 0.0), (3.0, 1000000, 0.99, 0.001), (0.7, 64, 0.5, 0.0),
]


def _tokens_of(stdout, with_logprobs=True):
    seqs = {}
    for line in stdout.splitlines():
        if line.startswith("@token"):
            f = dict(kv.split("=", 1) for kv in line.replace('top="', "top=").rstrip('"').split(" ", 5)[1:] if "=" in kv)
            seqs.setdefault(int(f.get("seq", 0)), []).append(int(f["id"].split()[0]))
    return [seqs[k] for k in sorted(seqs)]


def sampler_record(src, work):
    from conftest import SAMPLER_ROWS, SAMPLER_VOCAB, sampler_logits
    logits = sampler_logits()
    path = os.path.join(work, "logits.f32")
    logits.tofile(path)
    with open(os.path.join(work, "harness.c"), "w") as f:
        f.write(HARNESS)
    exe = os.path.join(work, "harness")
    subprocess.run(["cc", "-std=c99", "-O2", "-ffp-contract=off", "-I", os.path.join(src, "src"), "-o", exe,
                    os.path.join(work, "harness.c"), os.path.join(src, "src", "sample.o"),
                    os.path.join(src, "src", "mathx.o"), os.path.join(src, "src", "mem.o"), "-lm"], check=True)
    lines, keys = [], []
    for seed in (0, 1, 5, 0xDEADBEEF, 2 ** 64 - 1):
        lines.append(f"rng {seed} 6")
        keys.append(("rng", seed))
    for row in range(SAMPLER_ROWS):
        for si, (t, k, p, mp) in enumerate(SAMPLER_SETTINGS):
            seed = 1000 * row + si
            lines.append(f"pick {seed} {t} {k} {p} {mp} {row} 12")
            keys.append(("pick", seed, t, k, p, mp, row))
    r = subprocess.run([exe, path, str(SAMPLER_VOCAB), str(SAMPLER_ROWS)], input="\n".join(lines) + "\n",
                       capture_output=True, text=True, check=True)
    out = r.stdout.strip().splitlines()
    assert len(out) == len(keys)
    record = {"vocab": SAMPLER_VOCAB, "rows": SAMPLER_ROWS, "rng": [], "picks": []}
    for key, line in zip(keys, out):
        if key[0] == "rng":
            record["rng"].append({"seed": key[1], "uniforms": [float(x) for x in line.split()]})
        else:
            _, seed, t, k, p, mp, row = key
            record["picks"].append({"seed": seed, "temp": t, "top_k": k, "top_p": p, "min_p": mp, "row": row,
                                    "tokens": [int(x) for x in line.split()]})
    with open(os.path.join(HERE, "sampler.json"), "w") as f:
        json.dump(record, f, indent=None, separators=(",", ":"))
    print(f"sampler: {len(record['picks'])} settings x rows recorded")


def main(ref_dir):
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors
    from hfcpu_b200.weights.gguf import write_gguf
    work = tempfile.mkdtemp()
    src = os.path.join(work, "ref")
    shutil.copytree(ref_dir, src)
    subprocess.run(["make", "-C", src, "hfcpu"], check=True, stdout=subprocess.DEVNULL)
    # sharpness of attention: larger query/key weights make single scores stand out, and make the reference's
    # float16 cache show more; B's larger head size gets the smaller factor
    sampler_record(src, work)
    for name, lengths, n_new, sharp, extra in (("A", [7, 33, 70], 8, 4.0, {}), ("B", [1, 19, 60], 6, 2.0, {}),
                                               ("A_rope8", [7, 33, 70], 8, 4.0, {"rope_dim": 8})):
        cfg_d = dict(TINY[name[0]], use_sliding_window=False, **extra)
        cfg = config_from_dict(cfg_d)
        tensors = random_tensors(build_model_specs(cfg), 100 + ord(name[0]), torch.float32, std=0.05)
        for k in tensors:
            if ".q_proj." in k or ".k_proj." in k:
                tensors[k] = tensors[k] * sharp
        gguf = os.path.join(work, f"{name}.gguf")
        write_gguf(gguf, cfg_d, tensors)
        record = {"config": cfg_d, "seed": 100 + ord(name[0]), "std": 0.05, "sharp": sharp, "cases": []}
        for ids in make_requests(name[0], lengths, seed=77).values():
            r = subprocess.run([os.path.join(src, "hfcpu"), "--stdin-mode", "none", "--op", "generate", "--model", gguf,
                                "--prompt-ids", " ".join(map(str, ids)), "--temp", "0", "--max-tokens", str(n_new),
                                "--logprobs", "5", "--threads", "1"], capture_output=True, text=True, check=True)
            toks = []
            for line in r.stdout.splitlines():
                if line.startswith("@token"):
                    f = dict(kv.split("=", 1) for kv in line.replace('top="', "top=").rstrip('"').split(" ", 4)[1:])
                    top = [[int(a.split(":")[0]), float(a.split(":")[1])] for a in f["top"].split()]
                    toks.append({"id": int(f["id"]), "logprob": float(f["logprob"]), "top": top})
            record["cases"].append({"prompt": ids, "tokens": toks})
        if not extra:
            record["sampled"] = []
            ids = list(make_requests(name, lengths, seed=77).values())[1]
            for run in SAMPLED_RUNS:
                r = subprocess.run([os.path.join(src, "hfcpu"), "--stdin-mode", "none", "--op", "generate", "--model", gguf,
                                    "--prompt-ids", " ".join(map(str, ids)), "--temp", str(run["temp"]), "--top-k",
                                    str(run["top_k"]), "--top-p", str(run["top_p"]), "--min-p", str(run["min_p"]),
                                    "--seed", str(run["seed"]), "--n", str(run["n"]), "--max-tokens", "24",
                                    "--threads", "1"], capture_output=True, text=True, check=True)
                record["sampled"].append(dict(run, prompt=ids, sequences=_tokens_of(r.stdout)))
        with open(os.path.join(HERE, f"tiny_{name}.json"), "w") as f:
            json.dump(record, f, indent=1)
        print(f"tiny_{name}: {sum(len(c['tokens']) for c in record['cases'])} tokens recorded")
    shutil.rmtree(work)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py PATH_OF_THE_HFCPU_SOURCE_TREE")
    main(sys.argv[1])
