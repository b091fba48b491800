"""Build ``libqmm.so`` (the C-ABI kernel library) in-tree with nvcc for sm_100a.

    python -m jax_metallib_b200.build [--force]

nvcc cross-compiles without a GPU.  Objects go to ``csrc/build/``; the shared
library is written next to this file so that it travels with the source tree.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libqmm.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libqmm.so cannot be built")
    return exe


def sources() -> list[str]:
    out = []
    for root, _dirs, files in os.walk(CSRC):
        if os.path.basename(root) == "build":
            continue
        for f in sorted(files):
            if f.endswith((".cu", ".cc")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _headers_mtime() -> float:
    latest = 0.0
    for root, _dirs, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cuh", ".h", ".hpp")):
                latest = max(latest, os.path.getmtime(os.path.join(root, f)))
    inc = os.path.join(os.path.dirname(HERE), "include")
    for f in os.listdir(inc):
        latest = max(latest, os.path.getmtime(os.path.join(inc, f)))
    return latest


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    hdr = _headers_mtime()
    jobs = []
    objs = []
    for src in sources():
        rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(OBJ, os.path.splitext(rel)[0] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("QMM_EXTRA_NVCC_FLAGS", "").split(), "-x", "cu", "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(run, jobs):
                if verbose and log:
                    print(log)
    if jobs or not os.path.exists(LIB) or force:
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC", "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
        run(cmd)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
