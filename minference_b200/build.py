"""Compile the CUDA sources of this package into ``libminfer_b200.so`` (sm_100a only).

``python -m minference_b200.build`` or ``build()``; the library is written next to this file
so that it travels with the source tree.  nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libminfer_b200.so")
SOURCES = ["cabi.cu", "vs_index.cu", "sparse_attn_fwd.cu", "vs_estimate.cu", "block_sparse_index.cu", "block_mask_plan.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newest_source_mtime() -> float:
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


LIB_BOUNDS = os.path.join(HERE, "libminfer_b200_bounds.so")


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> str:
    """``bounds=True`` builds the range-checked debug variant (``-DMINF_BOUNDS``) as ``libminfer_b200_bounds.so``;
    set ``MINFER_B200_LIB`` to its path to make the package load it."""
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    lib = LIB_BOUNDS if bounds else LIB
    if not force and os.path.exists(lib) and os.path.getmtime(lib) >= _newest_source_mtime():
        return lib
    objs = []
    procs = []
    for s in srcs:
        o = s[:-3] + (".bounds.o" if bounds else ".o")
        objs.append(o)
        cmd = [_nvcc(), *NVCC_FLAGS, *(["-DMINF_BOUNDS"] if bounds else []), "-c", s, "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(out)
        elif verbose:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([_nvcc(), "-shared", "-o", lib, *objs, "-cudart", "static"])
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, bounds="--bounds" in sys.argv))
