"""Compiles the CUDA sources for sm_100a into one shared library, in the package folder.

Nothing is compiled at install time: the first call that needs the library builds it with nvcc
(one process per source file, in parallel), prints a line now and then while it waits, and
later calls find the finished library by the hash of the sources and flags.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import time
from typing import List

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG_DIR, "csrc")
OUT_DIR = os.path.join(PKG_DIR, "_native")
LIB_NAME = "libhfb200.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _flags() -> List[str]:
    """The fixed flags plus what HFB_NVCC_EXTRA adds (for instance -DHFB_TRACE for the kernel timeline)."""
    return NVCC_FLAGS + os.environ.get("HFB_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                       "the CUDA kernels of this package cannot be built")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(_flags()).encode())
    return h.hexdigest()[:16]


def library_path() -> str:
    return os.path.join(OUT_DIR, LIB_NAME)


def is_current() -> bool:
    stamp = os.path.join(OUT_DIR, "stamp")
    try:
        with open(stamp) as f:
            return f.read().strip() == _digest() and os.path.exists(library_path())
    except OSError:
        return False


def build(verbose: bool = True, force: bool = False) -> str:
    """Build the library if it is missing or stale; returns its path."""
    if not force and is_current():
        return library_path()
    nvcc = _nvcc()
    build_dir = os.path.join(OUT_DIR, "_build")
    os.makedirs(build_dir, exist_ok=True)
    say = (lambda m: print(f"[hfcpu_b200] {m}", file=sys.stderr, flush=True)) if verbose else (lambda m: None)
    srcs = sources()
    say(f"compiling {len(srcs)} CUDA sources for sm_100a with {nvcc} (first use; this takes a minute or two)")
    t0 = time.time()
    procs = []
    for f in srcs:
        obj = os.path.join(build_dir, f[:-3] + ".o")
        cmd = [nvcc, *_flags(), "-I", CSRC, "-c", os.path.join(CSRC, f), "-o", obj]
        procs.append((f, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    pending = list(procs)
    last = time.time()
    while pending:
        for item in list(pending):
            f, obj, p = item
            if p.poll() is not None:
                pending.remove(item)
                out = p.stdout.read()
                if p.returncode != 0:
                    for _, _, q in pending:
                        q.kill()
                    raise RuntimeError(f"nvcc failed on {f}:\n{out}")
                say(f"  compiled {f} ({time.time() - t0:.0f} s)")
        if pending:
            time.sleep(0.2)
            if time.time() - last > 10:
                say(f"  still compiling: {', '.join(x[0] for x in pending)} ({time.time() - t0:.0f} s)")
                last = time.time()
    tmp = library_path() + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *[o for _, o, _ in procs], "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-cudart", "static"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{r.stdout}")
    os.replace(tmp, library_path())
    with open(os.path.join(OUT_DIR, "stamp"), "w") as f:
        f.write(_digest())
    say(f"built {library_path()} in {time.time() - t0:.0f} s")
    return library_path()


if __name__ == "__main__":
    build(force="--force" in sys.argv)
