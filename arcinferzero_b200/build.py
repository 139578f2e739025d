"""Builds libizb200.so (the CUDA library behind include/izb200.h) in-tree with nvcc for sm_100a.

    python -m arcinferzero_b200.build [--verbose]

nvcc cross-compiles without a GPU.  Objects are cached under arcinferzero_b200/csrc/build/ and rebuilt when a source
or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libizb200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fopenmp",
         "-ccbin", "/usr/bin/g++"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def build(verbose: bool = False) -> str:
    os.makedirs(os.path.join(CSRC, "build"), exist_ok=True)
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")] + [
        os.path.join(os.path.dirname(HERE), "include", "izb200.h")]
    newest_hdr = max(os.path.getmtime(h) for h in hdrs)
    objs, jobs = [], []
    for s in sources():
        src, obj = os.path.join(CSRC, s), os.path.join(CSRC, "build", s[:-3] + ".o")
        objs.append(obj)
        if not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_hdr):
            jobs.append([NVCC, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for log in ex.map(run, jobs):
            if verbose and log:
                print(log)
    if jobs or not os.path.exists(OUT):
        run([NVCC, "-shared", "-o", OUT, *objs, "-lcudart", "-ldl", "-lgomp", "-ccbin", "/usr/bin/g++"])
    return OUT


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv))
