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
    for name, lengths, n_new, sharp in (("A", [7, 33, 70], 8, 4.0), ("B", [1, 19, 60], 6, 2.0)):
        cfg_d = dict(TINY[name], use_sliding_window=False)
        cfg = config_from_dict(cfg_d)
        tensors = random_tensors(build_model_specs(cfg), 100 + ord(name), torch.float32, std=0.05)
        for k in tensors:
            if ".q_proj." in k or ".k_proj." in k:
                tensors[k] = tensors[k] * sharp
        gguf = os.path.join(work, f"{name}.gguf")
        write_gguf(gguf, cfg_d, tensors)
        record = {"config": cfg_d, "seed": 100 + ord(name), "std": 0.05, "sharp": sharp, "cases": []}
        for ids in make_requests(name, lengths, seed=77).values():
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
        with open(os.path.join(HERE, f"tiny_{name}.json"), "w") as f:
            json.dump(record, f, indent=1)
        print(f"tiny_{name}: {sum(len(c['tokens']) for c in record['cases'])} tokens recorded")
    shutil.rmtree(work)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py PATH_OF_THE_HFCPU_SOURCE_TREE")
    main(sys.argv[1])
