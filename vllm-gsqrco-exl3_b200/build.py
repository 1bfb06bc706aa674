"""Build the C-ABI shared library `gsq_b200/libgsq.so` from csrc/*.cu for sm_100a with nvcc.

    python vllm-gsqrco-exl3_b200/build.py [--force] [--verbose]

Each translation unit is compiled to an object in csrc/_build/ (in parallel, skipped when the
object is newer than every source and header), then linked with -shared. The library lives inside
the package directory so that it travels with the source tree.
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "gsq_b200", "libgsq.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "gsq.h"))
    hs.append(os.path.join(os.path.dirname(HERE), "include", "gsq_debug.h"))
    return hs


def build(force: bool = False, verbose: bool = False) -> str:
    tables = os.path.join(CSRC, "gsq_tables.h")
    if not os.path.exists(tables):
        subprocess.check_call([sys.executable, os.path.join(CSRC, "gen_tables.py")])
    bdir = os.path.join(CSRC, "_build")
    os.makedirs(bdir, exist_ok=True)
    newest_h = max(os.path.getmtime(h) for h in _headers())
    objs, jobs = [], []
    for src in _sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(bdir, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), newest_h):
            jobs.append([NVCC, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs)))) as ex:
        for log in ex.map(run, jobs):
            if verbose and log:
                print(log)
    if jobs or not os.path.exists(OUT):
        run([NVCC, "-shared", "-cudart", "static", "-o", OUT, *objs])
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
